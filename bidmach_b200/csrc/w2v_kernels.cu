// Word2Vec skip-gram negative-sampling minibatch kernels for sm_100a, and the
// C entry points that launch them.
//
// What the four kernels compute (A is indexed by centre / negative words and B
// by context words; both are dim x vocab fp32, word w = row [w*dim,(w+1)*dim)):
//
//   Pos      for every centre i with W[i] >= 0 and every offset j in
//            [LB[i], UB[i]], j != 0, 0 <= i+j < ncols, W[i+j] >= 0:
//              g = lrate * (1 - sigmoid(A[W[i]] . B[W[i+j]]))
//              A[W[i]]   += (1+W[i])^vexp   * g * B[W[i+j]]
//              B[W[i+j]] += (1+W[i+j])^vexp * g * A[W[i]]
//   Neg      for every column c and all j < nwa, k < nwb:
//              g = -lrate * sigmoid(A[WA[j,c]] . B[WB[k,c]])
//              A[WA[j,c]] += (1+WA[j,c])^vexp * g * B[WB[k,c]]
//              B[WB[k,c]] += (1+WB[k,c])^vexp * g * A[WA[j,c]]
//   EvalPos  Retval[0] += sum over the Pos pairs of log(max(sigmoid(a.b), 1e-20))
//   EvalNeg  Retval[0] += sum over the Neg pairs of log(max(1 - sigmoid(a.b), 1e-20))
//
// These are the semantics of __word2vecPos / __word2vecNeg / __word2vecEvalPos /
// __word2vecEvalNeg (jni/src/DNN127.cu:20-188, 546-667, 195-325, 831-930) and of
// their CPU twins (jni/src/BIDMach_CPUMACH.c:10-78, 186-264, 368-483).
//
// Update-conflict policy: hogwild with atomics.  All gradients of one centre
// (Pos) or one column (Neg) are computed from the row values read at the start
// of that unit of work; the deltas are then added with 128-bit atomic
// reductions, so concurrent units that touch the same row never lose an
// update, but may read a row before or after another unit's delta landed.  On
// inputs where no row is shared between units the result equals the sequential
// CPU result up to fp32 summation order.
//
// Work decomposition: a warp per stretch of token positions (Pos) or per column
// (Neg); a row is dim/4 16-byte vectors of which lane l owns l, l+32, ...; dot
// products are reduced with warp shuffles so that each total ends on one lane;
// grids are sized to fill every SM.  Neg stages a column's rows in shared memory
// with bulk asynchronous copies and is bound by the L2's atomic throughput; the
// scoring kernels read rows straight from global memory.
//
// Pos walks the minibatch in order: every warp owns a contiguous stretch of
// positions and visits its centres one after the other.  The delta of a
// context row is not sent to memory per pair; it is accumulated in a ring of
// 2*skip+1 row-sized slots in shared memory (one per position of the sliding
// window, private to the warp) and added to B once, when the window has moved
// past that position.  Each position therefore costs two atomic row updates
// (its A row as a centre, its B row as a context) instead of one per pair, and
// a pair is still evaluated by exactly one warp from one reading of its rows.
//
// Hot rows: under a Zipf-like draw a handful of word ids receive a large share
// of all updates, and atomic adds to one address serialise in L2.  Updates to
// the most frequent ids (id + 1 < 2^levels, 15 ids by default; ids are
// frequency ranks) are therefore spread over replica rows in a small side
// buffer (16 for id 0, 8 for ids 1-2, 4 for ids 3-6, 2 for ids 7-14).  While
// the update kernel runs, every warp periodically moves the contents of one
// replica row into the model ("continuous folding"), so that readers of a hot
// row see its updates within microseconds, as they would with plain atomics;
// a tiny kernel folds what is left after the update kernel.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <type_traits>

#include "w2v_device.cuh"
#include "w2v_internal.h"
#include "w2v_rows.cuh"

namespace w2v {

constexpr int kPosThreads = 128;
constexpr int kNegThreads = 128;
constexpr int kGenericThreads = 128;

// ---------------------------------------------------------------------------
// Positive pairs
// ---------------------------------------------------------------------------

// Lane `l` looks at window offset LB+l of centre i.  Returns the context word
// there or -1 when that offset yields no pair.
__device__ __forceinline__ int window_word(const int *__restrict__ W, int i, int lb, int ub,
                                           int ncols, int lane) {
  int j = lb + lane;
  if (j > ub || j == 0) return -1;
  int t = i + j;
  if (t < 0 || t >= ncols) return -1;
  return W[t];
}

// Folding period for this launch.  Updates to a hot row sit in its replicas until
// the next fold, and everything computed meanwhile uses the row without them.  If the
// most frequent word takes a share p0 of the text, `per_unit` updates of it arrive per
// unit of work (column / position), its replica rows come round every `cycled` folds
// and each update moves the row by about `rate`, then fold_every units between a
// warp's folds leave per_unit * p0 * cycled * fold_every * rate worth of updates unseen.
// Measured on unsubsampled Zipf(1.07) text: training is as stable as with plain atomics
// while that product stays near 0.1 and diverges from about 0.4; at the reference's
// default subsampling (p0 about 0.01) the configured period already satisfies it.
__device__ __forceinline__ int fold_period(const HotRows &hot, float rate, float per_unit) {
  int fe = hot.fold_every;
  if (fe > 0 && hot.stats != nullptr) {
    const float kept = (float)max(1, hot.stats[0]);
    const float p0 = (float)hot.stats[1] / kept;
    // replica rows of the most frequent word come round every `cycled` turns (fold_one_replica)
    const float cycled = (hot.limit > 2 ? 4.0f : 2.0f) * (float)hot.rmax;
    const float unseen_per_fold = per_unit * p0 * cycled * fabsf(rate);
    if (unseen_per_fold * (float)fe > 0.1f) fe = max(4, (int)(0.1f / unseen_per_fold));
  }
  return fe;
}

template <int NR>
__device__ __forceinline__ void row_red_to(float *p, int nvec, int lane, const Row<NR> &r) {
#pragma unroll
  for (int q = 0; q < NR; q++) {
    int idx = lane + 32 * q;
    if (idx < nvec) red_add_v4(p + 4 * idx, r.v[q]);
  }
}

// Continuous folding.  Every so often a warp takes one replica row (the next
// of the schedule in fold_one_replica), atomically swaps its contents for zeros and adds
// what it took to the model row the replica stands for.  Replicas therefore
// hold only the last few microseconds of updates, and readers of a hot row see
// its updates almost as soon as they would without replicas; what is left at
// the end of the kernel is collected by hot_fold_kernel.
__device__ __forceinline__ void exch_zero_v4(float *addr, u64 &lo, u64 &hi) {
  // two 64-bit exchanges: every float is independent, so 8-byte atomicity is enough
  lo = atomicExch(reinterpret_cast<u64 *>(addr), 0ull);
  hi = atomicExch(reinterpret_cast<u64 *>(addr) + 1, 0ull);
}

template <int NR>
__device__ __forceinline__ void fold_one_replica(const HotRows &hot, float *A, float *B, int dim,
                                                 int nvec, int lane, unsigned turn) {
  // Matrices alternate.  Level L (ids 2^L - 1 .. 2^(L+1) - 2, rmax replica rows in all)
  // takes the turns with exactly L trailing one bits, i.e. a share 2^-(L+1), and the last
  // level the remainder: an id's replicas come round in proportion to how often a word of
  // its rank occurs (1 / rank), so every hot row carries about the same unseen amount.
  const int levels = 31 - __clz(hot.limit);
  const bool in_b = turn & 1u;
  const unsigned u = turn >> 1;
  const int ones = __ffs((int)~u) - 1;  // trailing one bits of u (-1 when all are set)
  const int lv = (ones < 0 || ones > levels - 1) ? levels - 1 : ones;
  const unsigned k = u >> min(lv + 1, levels - 1);
  const int row = lv * hot.rmax + (int)(k % (unsigned)hot.rmax);
  const int reps = hot.rmax >> lv;
  const int id = (1 << lv) - 1 + (row - lv * hot.rmax) / reps;
  float *src = (in_b ? hot.shadowB : hot.shadowA) + (int64_t)row * dim;
  float *dst = (in_b ? B : A) + (int64_t)id * dim;
  // all exchanges first, so that their round trips overlap
  u64 got[NR][2];
#pragma unroll
  for (int q = 0; q < NR; q++) {
    const int idx = lane + 32 * q;
    got[q][0] = got[q][1] = 0ull;
    if (idx < nvec) exch_zero_v4(src + 4 * idx, got[q][0], got[q][1]);
  }
#pragma unroll
  for (int q = 0; q < NR; q++) {
    const int idx = lane + 32 * q;
    if (idx < nvec && (got[q][0] | got[q][1])) {  // untouched replicas (also of ids beyond the vocabulary) stay out of the model
      float4 v;
      unpack2(got[q][0], v.x, v.y);
      unpack2(got[q][1], v.z, v.w);
      red_add_v4(dst + 4 * idx, v);
    }
  }
}

// Folds the replica rows of the hot ids back into the model and clears them.
// grid = (hot ids, 2 matrices).
__global__ void hot_fold_kernel(int dim, HotRows hot, float *A, float *B) {
  const int h = blockIdx.x;
  float *M = blockIdx.y ? B : A;
  float *S = blockIdx.y ? hot.shadowB : hot.shadowA;
  const int level = 31 - __clz(h + 1);
  const int reps = hot.rmax >> level;
  float *base = S + (int64_t)(hot.rmax * level + (h + 1 - (1 << level)) * reps) * dim;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float sum = 0.f;
    for (int r = 0; r < reps; r++) {
      sum += base[(int64_t)r * dim + c];
      base[(int64_t)r * dim + c] = 0.f;
    }
    if (sum != 0.f) M[(int64_t)h * dim + c] += sum;  // ids that were never touched are not read
  }
}

// Neighbour rows loaded and reduced together: as many as the register file
// allows for rows of NR vectors per lane.
template <int NR>
struct ChunkOf {
  static constexpr int value = NR <= 4 ? 5 : (NR <= 6 ? 3 : 2);
};
// The scoring kernel holds no deltas, so it can take more rows at a time.
template <int NR>
struct EvalChunkOf {
  static constexpr int value = NR <= 3 ? 10 : ChunkOf<NR>::value;
};
// Resident blocks per SM the positive update is compiled for (its ring of
// row-sized slots in shared memory allows no more for wide rows anyway).
template <int NR>
struct PosBlocksOf {
  static constexpr int value = NR <= 3 ? 4 : (NR <= 5 ? 2 : 1);
};

// Calls take(integral_constant<n>) for a run-time n in [LO, HI]: one
// instantiation of the chunk body per size, exactly one of them taken.
template <int LO, int HI, class F>
__device__ __forceinline__ void take_n(int n, F &take) {
  if constexpr (LO <= HI) {
    if (n == LO)
      take(std::integral_constant<int, LO>());
    else
      take_n<LO + 1, HI>(n, take);
  }
}

// What lane `lane` sees at offset lane - skip from position t: the word there
// and whether t, as a centre, pairs with it.
struct Neighbour {
  int word;
  bool t_is_centre;
};

__device__ __forceinline__ Neighbour look_at_neighbour(const int *__restrict__ W, int t, int lbt,
                                                       int ubt, int skip, int ncols, int lane) {
  Neighbour nb = {-1, false};
  const int j = lane - skip, u = t + j;
  if (lane <= 2 * skip && j != 0 && j >= lbt && j <= ubt && u >= 0 && u < ncols) {
    const int w = W[u];
    if (w >= 0) {
      nb.word = w;
      nb.t_is_centre = true;
    }
  }
  return nb;
}

// Which of the two positive-update kernels takes a launch: both are launched, both read the same
// count of valid words that the launch's preparation left on the device (HotRows::stats), and
// exactly one of them goes on.  With three quarters or more of the positions holding a word, two
// centres at a time pay (dense text: 1.44 against 1.54 ms on the benchmark's minibatches); on
// subsampled text, where many positions are empty and windows are short, one centre at a time
// with more resident warps does (0.77 against 0.78 ms).
__device__ __forceinline__ bool pos_text_is_dense(const HotRows &hot, int ncols) {
  return hot.stats != nullptr && 4ll * hot.stats[0] >= 3ll * ncols;
}

// Shared memory: per warp, (2*skip+1) slots of nvec float4 (one context-row
// delta each), all zero whenever they hold nothing.  Lane l only ever touches
// elements l, l+32, ... of a slot, so no synchronisation is needed between the
// lanes of the owning warp.
// SLICED: W holds global ids and A / B the rows of one vocabulary slice (SliceMap): a word
// without a row here is skipped like a masked one, head-head pairs and writes to head rows
// follow the slice's do_head (word2vecPosSlice, BIDMach_CPUMACH.c:90-184).
template <int NR, bool SLICED>
__global__ void __launch_bounds__(kPosThreads, PosBlocksOf<NR>::value)
    pos_update_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                      const int *__restrict__ W, const int *__restrict__ LB,
                      const int *__restrict__ UB, float *A, float *B, float lrate, float vexp,
                      HotRows hot, SliceMap sl, int yield_dense) {
  constexpr int kChunk = ChunkOf<NR>::value;
  extern __shared__ ulonglong2 ring_storage[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = dim >> 2;
  const bool tail = lane + 32 * (NR - 1) < nvec;
  const int slots = 2 * skip + 1;
  ulonglong2 *ring = ring_storage + (size_t)warp * slots * nvec + lane;  // this lane's part of slot 0
  const unsigned gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  // dense text goes to pos_update_pair_kernel, launched beside this one (see there)
  if (yield_dense && pos_text_is_dense(hot, ncols)) return;
  const int per_warp = (ncols + (int)nwarps - 1) / (int)nwarps;
  const int first = (int)gwarp * per_warp;
  const int last = min(ncols, first + per_warp);
  unsigned dirty = 0;             // bit s: slot s holds a pending delta
  for (int s = 0; s < slots; s++) {
#pragma unroll
    for (int q = 0; q < NR; q++)
      if (vec_ok<NR>(q, tail)) ring[s * nvec + 32 * q] = make_ulonglong2(0ull, 0ull);
  }

  // Slot of position t - skip, the oldest position of the current window; it
  // advances by one per position, so no division is needed to find a slot.
  int wslot = 0;
  // B[W[u]] += the given slot (which belongs to position u), if it holds
  // anything; the slot is left zeroed for the position that takes it next
  auto retire = [&](int wu, int slot) {  // wu = the word at the slot's position
    if ((dirty >> slot) & 1u) {
      dirty &= ~(1u << slot);
      float *dst = update_target(B, hot.shadowB, hot, wu, dim, gwarp) + 4 * lane;
      ulonglong2 *sp = ring + slot * nvec;
#pragma unroll
      for (int q = 0; q < NR; q++) {
        if (vec_ok<NR>(q, tail)) {
          red_add_v4(dst + 128 * q, *reinterpret_cast<const float4 *>(sp + 32 * q));
          sp[32 * q] = make_ulonglong2(0ull, 0ull);
        }
      }
    }
  };
  // about six pairs per position; the rate of the positive update is five times the negative one's
  const int fold_every = 2 * fold_period(hot, lrate, 6.0f);
  int until_fold = fold_every;
  unsigned fold_turn = gwarp * 3u;

  // The index data of a position (its window of words, lane l holding offset l - skip, and
  // its bounds) is fetched one position ahead, so that the row loads of a position do not
  // wait for a chain of dependent index loads first.
  auto fetch = [&](int t, int &wraw, int &lbt, int &ubt) {
    const int u = t + lane - skip;
    const bool in = t < last;
    wraw = (in && lane <= 2 * skip && u >= 0 && u < ncols) ? W[u] : -1;
    if (SLICED) wraw = sl.local(wraw);
    lbt = in ? max(LB[t], -skip) : 0;
    ubt = in ? min(UB[t], skip) : 0;
  };
  int wraw, lbt, ubt;
  fetch(first, wraw, lbt, ubt);

  for (int t = first; t < last; t++) {
    int wraw_next, lb_next, ub_next;
    fetch(t + 1, wraw_next, lb_next, ub_next);
    const int wt = __shfl_sync(kFullMask, wraw, skip);
    const int w_oldest = __shfl_sync(kFullMask, wraw, 0);  // the word at position t - skip
    if (wt >= 0) {
      Neighbour nb = {-1, false};
      {
        const int j = lane - skip;
        bool pair = j != 0 && j >= lbt && j <= ubt && wraw >= 0;
        if (SLICED && sl.skips_head_pairs() && wt < sl.nhead && wraw < sl.nhead) pair = false;
        if (pair) {
          nb.word = wraw;
          nb.t_is_centre = true;
        }
      }
      unsigned todo = __ballot_sync(kFullMask, nb.t_is_centre);
      if (todo) {
        // lane 31 never carries a neighbour (at most 31 offsets), so it
        // evaluates the centre's scale while the others do their context's
        const int sid = (lane == 31) ? wt : nb.word;
        const float sc = (sid >= 0) ? freq_scale(SLICED ? sl.global(sid) : sid, vexp) : 0.f;
        const float sa = __shfl_sync(kFullMask, sc, 31);
        PRow<NR> a, da;
        prow_load_lane(a, reinterpret_cast<const ulonglong2 *>(A + (int64_t)wt * dim) + lane, tail);
        prow_zero(da);
        // CH contexts at a time: their rows are loaded together, the CH dot
        // products are reduced together and one lane each evaluates a sigmoid
        auto take = [&](auto width) {
          constexpr int CH = decltype(width)::value;
          static_assert(Spread<CH>::FIN == 1, "one total per lane expected");
          int src[CH];
          int wc[CH];
          PRow<NR> rows[CH];
          float p[CH];
#pragma unroll
          for (int c = 0; c < CH; c++) {
            src[c] = __ffs(todo) - 1;
            todo &= todo - 1;
            wc[c] = __shfl_sync(kFullMask, nb.word, src[c]);
            prow_load_lane(rows[c], reinterpret_cast<const ulonglong2 *>(B + (int64_t)wc[c] * dim) + lane, tail);
          }
#pragma unroll
          for (int c = 0; c < CH; c++) p[c] = prow_dot_partial(a, rows[c]);
          Spread<CH>::reduce(p, lane);
          const float mine = lrate * (1.0f - sigmoid_guard(p[0]));
#pragma unroll
          for (int c = 0; c < CH; c++) {
            const float g = __shfl_sync(kFullMask, mine, Spread<CH>::lane_of(c));
            const float sb = __shfl_sync(kFullMask, sc, src[c]);
            prow_axpy(da, sa * g, rows[c]);
            if (SLICED && sl.freezes_head() && wc[c] < sl.nhead) continue;  // head rows are read-only
            // context side: slot(u) += (sb * g) * a
            int slot = wslot + src[c];  // position t - skip + src[c]
            if (slot >= slots) slot -= slots;
            ulonglong2 *sp = ring + slot * nvec;
            const u64 coef = pack2(sb * g, sb * g);
            dirty |= 1u << slot;
#pragma unroll
            for (int q = 0; q < NR; q++) {
              if (vec_ok<NR>(q, tail)) {
                ulonglong2 v = sp[32 * q];
                v.x = fma2(coef, a.v[q][0], v.x);
                v.y = fma2(coef, a.v[q][1], v.y);
                sp[32 * q] = v;
              }
            }
          }
        };
        // a window larger than one chunk is split evenly (6 contexts as 3 + 3, not 5 + 1)
        int cnt = __popc(todo);
        while (cnt > 0) {
          const int n = cnt > kChunk ? min(kChunk, (cnt + 1) >> 1) : cnt;
          cnt -= n;
          take_n<1, kChunk>(n, take);
        }
        if (!(SLICED && sl.freezes_head() && wt < sl.nhead))
          prow_red_lane(update_target(A, hot.shadowA, hot, wt, dim, gwarp) + 4 * lane, tail, da);
      }
    }
    // no later centre of this warp reaches position t - skip
    if (dirty) retire(w_oldest, wslot);
    wslot = (wslot + 1 == slots) ? 0 : wslot + 1;
    if (fold_every > 0 && --until_fold == 0) {
      until_fold = fold_every;
      fold_one_replica<NR>(hot, A, B, dim, nvec, lane, fold_turn++);
    }
    wraw = wraw_next;
    lbt = lb_next;
    ubt = ub_next;
  }
  for (int k = 0; k < slots && dirty; k++) {  // positions last - skip ... last + skip
    const int u = last - skip + k;
    // a dirty slot belongs to a position inside the minibatch that holds a word
    int wu = (u >= 0 && u < ncols) ? W[u] : 0;
    if (SLICED) wu = sl.local(wu);
    retire(wu, wslot);
    wslot = (wslot + 1 == slots) ? 0 : wslot + 1;
  }
}

// Two centres at a time.  Positions t and t + 1 share most of their windows, so a context row
// that both take is loaded once, meets both centre rows in one pass and its ring slot is updated
// once for both: fewer loads and fewer shared-memory read-modify-writes per position than with
// one centre at a time, paid for with two centre rows and two centre deltas in registers (168
// registers per thread, 12 warps per SM).  Lane l stands for position t - skip + l of the
// 2*skip + 2 positions the two windows span; the ring has as many slots.
template <int NR>
struct PairChunkOf {
  static constexpr int value = NR <= 3 ? 5 : (NR <= 4 ? 3 : 2);
};

template <int NR>
__global__ void __launch_bounds__(kPosThreads, 3)
    pos_update_pair_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                           const int *__restrict__ W, const int *__restrict__ LB,
                           const int *__restrict__ UB, float *A, float *B, float lrate, float vexp,
                           HotRows hot) {
  constexpr int kChunk = PairChunkOf<NR>::value;
  extern __shared__ ulonglong2 ring_storage[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = dim >> 2;
  const bool tail = lane + 32 * (NR - 1) < nvec;
  const int slots = 2 * skip + 2;
  ulonglong2 *ring = ring_storage + (size_t)warp * slots * nvec + lane;  // this lane's part of slot 0
  const unsigned gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  if (!pos_text_is_dense(hot, ncols)) return;   // pos_update_kernel takes the launch
  // stretches of an even number of positions, so that every warp starts on a pair
  const int per_warp = (((ncols + (int)nwarps - 1) / (int)nwarps) + 1) & ~1;
  const int first = (int)min((long long)gwarp * per_warp, (long long)ncols);
  const int last = min(ncols, first + per_warp);
  unsigned dirty = 0;             // bit s: slot s holds a pending delta
  for (int s = 0; s < slots; s++) {
#pragma unroll
    for (int q = 0; q < NR; q++)
      if (vec_ok<NR>(q, tail)) ring[s * nvec + 32 * q] = make_ulonglong2(0ull, 0ull);
  }
  int wslot = 0;  // slot of position t - skip
  auto retire = [&](int wu, int slot) {  // wu = the word at the slot's position
    if ((dirty >> slot) & 1u) {
      dirty &= ~(1u << slot);
      float *dst = update_target(B, hot.shadowB, hot, wu, dim, gwarp) + 4 * lane;
      ulonglong2 *sp = ring + slot * nvec;
#pragma unroll
      for (int q = 0; q < NR; q++) {
        if (vec_ok<NR>(q, tail)) {
          red_add_v4(dst + 128 * q, *reinterpret_cast<const float4 *>(sp + 32 * q));
          sp[32 * q] = make_ulonglong2(0ull, 0ull);
        }
      }
    }
  };
  const int fold_every = 2 * fold_period(hot, lrate, 6.0f);
  int until_fold = fold_every;
  unsigned fold_turn = gwarp * 3u;

  // index data of the pair (t, t + 1), fetched one pair ahead
  auto fetch = [&](int t, int &wraw, int &lb0, int &ub0, int &lb1, int &ub1) {
    const int u = t + lane - skip;
    wraw = (t < last && lane < slots && u >= 0 && u < ncols) ? W[u] : -1;
    const bool in0 = t < last, in1 = t + 1 < last;
    lb0 = in0 ? max(LB[t], -skip) : 0;
    ub0 = in0 ? min(UB[t], skip) : 0;
    lb1 = in1 ? max(LB[t + 1], -skip) : 0;
    ub1 = in1 ? min(UB[t + 1], skip) : 0;
  };
  int wraw, lb0, ub0, lb1, ub1;
  fetch(first, wraw, lb0, ub0, lb1, ub1);

  for (int t = first; t < last; t += 2) {
    int wraw_n, lb0_n, ub0_n, lb1_n, ub1_n;
    fetch(t + 2, wraw_n, lb0_n, ub0_n, lb1_n, ub1_n);
    const int wt0 = __shfl_sync(kFullMask, wraw, skip);
    const int wt1 = (t + 1 < last) ? __shfl_sync(kFullMask, wraw, skip + 1) : -1;
    const int w_old0 = __shfl_sync(kFullMask, wraw, 0), w_old1 = __shfl_sync(kFullMask, wraw, 1);
    const int j0 = lane - skip, j1 = lane - skip - 1;
    const bool pair0 = wt0 >= 0 && wraw >= 0 && j0 != 0 && j0 >= lb0 && j0 <= ub0;
    const bool pair1 = wt1 >= 0 && wraw >= 0 && j1 != 0 && j1 >= lb1 && j1 <= ub1;
    const unsigned m0 = __ballot_sync(kFullMask, pair0), m1 = __ballot_sync(kFullMask, pair1);
    unsigned todo = m0 | m1;
    if (todo) {
      // every lane that holds a word evaluates its scale: the centres' lanes among them
      const float sc = (wraw >= 0) ? freq_scale(wraw, vexp) : 0.f;
      const float sa0 = __shfl_sync(kFullMask, sc, skip), sa1 = __shfl_sync(kFullMask, sc, skip + 1);
      PRow<NR> a0, a1, da0, da1;
      prow_zero(a0);
      prow_zero(a1);
      if (m0) prow_load_lane(a0, reinterpret_cast<const ulonglong2 *>(A + (int64_t)wt0 * dim) + lane, tail);
      if (m1) prow_load_lane(a1, reinterpret_cast<const ulonglong2 *>(A + (int64_t)wt1 * dim) + lane, tail);
      prow_zero(da0);
      prow_zero(da1);
      auto take = [&](auto width) {
        constexpr int CH = decltype(width)::value;
        static_assert(Spread<2 * CH>::FIN == 1, "one total per lane expected");
        int src[CH];
        PRow<NR> rows[CH];
        float p[2 * CH];
#pragma unroll
        for (int c = 0; c < CH; c++) {
          src[c] = __ffs(todo) - 1;
          todo &= todo - 1;
          const int wc = __shfl_sync(kFullMask, wraw, src[c]);
          prow_load_lane(rows[c], reinterpret_cast<const ulonglong2 *>(B + (int64_t)wc * dim) + lane, tail);
        }
#pragma unroll
        for (int c = 0; c < CH; c++) {
          p[2 * c] = prow_dot_partial(a0, rows[c]);
          p[2 * c + 1] = prow_dot_partial(a1, rows[c]);
        }
        Spread<2 * CH>::reduce(p, lane);
        const float mine = lrate * (1.0f - sigmoid_guard(p[0]));
#pragma unroll
        for (int c = 0; c < CH; c++) {
          float g0 = __shfl_sync(kFullMask, mine, Spread<2 * CH>::lane_of(2 * c));
          float g1 = __shfl_sync(kFullMask, mine, Spread<2 * CH>::lane_of(2 * c + 1));
          if (!((m0 >> src[c]) & 1u)) g0 = 0.f;   // not a pair of this centre
          if (!((m1 >> src[c]) & 1u)) g1 = 0.f;
          const float sb = __shfl_sync(kFullMask, sc, src[c]);
          prow_axpy(da0, sa0 * g0, rows[c]);
          prow_axpy(da1, sa1 * g1, rows[c]);
          // context side, once for both centres: slot(u) += sb * (g0 * a0 + g1 * a1)
          int slot = wslot + src[c];
          if (slot >= slots) slot -= slots;
          ulonglong2 *sp = ring + slot * nvec;
          const u64 c0 = pack2(sb * g0, sb * g0), c1 = pack2(sb * g1, sb * g1);
          dirty |= 1u << slot;
#pragma unroll
          for (int q = 0; q < NR; q++) {
            if (vec_ok<NR>(q, tail)) {
              ulonglong2 v = sp[32 * q];
              v.x = fma2(c1, a1.v[q][0], fma2(c0, a0.v[q][0], v.x));
              v.y = fma2(c1, a1.v[q][1], fma2(c0, a0.v[q][1], v.y));
              sp[32 * q] = v;
            }
          }
        }
      };
      int cnt = __popc(todo);
      while (cnt > 0) {
        const int chunks = (cnt + kChunk - 1) / kChunk;
        const int n = (cnt + chunks - 1) / chunks;  // even split: 7 contexts as 4 + 3, not 4 + 3 + 0
        cnt -= n;
        take_n<1, kChunk>(n, take);
      }
      if (m0) prow_red_lane(update_target(A, hot.shadowA, hot, wt0, dim, gwarp) + 4 * lane, tail, da0);
      if (m1) prow_red_lane(update_target(A, hot.shadowA, hot, wt1, dim, gwarp) + 4 * lane, tail, da1);
    }
    // no later centre of this warp reaches positions t - skip and t - skip + 1
    if (dirty) {
      retire(w_old0, wslot);
      retire(w_old1, (wslot + 1 == slots) ? 0 : wslot + 1);
    }
    wslot += 2;
    if (wslot >= slots) wslot -= slots;
    if (fold_every > 0 && (until_fold -= 2) <= 0) {
      until_fold = fold_every;
      fold_one_replica<NR>(hot, A, B, dim, nvec, lane, fold_turn++);
    }
    wraw = wraw_n;
    lb0 = lb0_n;
    ub0 = ub0_n;
    lb1 = lb1_n;
    ub1 = ub1_n;
  }
  // what is left in the ring belongs to the positions from (end of the last pair) - skip on
  const int t_end = first + ((last - first + 1) & ~1);
  for (int k = 0; k < slots && dirty; k++) {
    const int u = t_end - skip + k;
    const int wu = (u >= 0 && u < ncols) ? W[u] : 0;
    retire(wu, wslot);
    wslot = (wslot + 1 == slots) ? 0 : wslot + 1;
  }
}

// Adds this block's double partial sum into scratch[0]; the block that
// arrives last moves the grand total into Retval[0] (one float add, as the
// reference accumulates into a caller-zeroed float) and re-arms the scratch.
__device__ __forceinline__ void finish_eval_sum(double lane_sum, EvalScratch *scratch,
                                                float *retval) {
  __shared__ double warp_part[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double s = warp_sum(lane_sum);
  if (lane == 0) warp_part[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int k = 0; k < (int)(blockDim.x >> 5); k++) tot += warp_part[k];
    atomicAdd(&scratch->sum, tot);
    __threadfence();
    unsigned ticket = atomicAdd(&scratch->arrived, 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      double total = atomicAdd(&scratch->sum, 0.0);
      atomicAdd(retval, (float)total);
      scratch->sum = 0.0;
      scratch->arrived = 0u;
      __threadfence();
    }
  }
}

// SLICED: pairs whose two words both have a row on this slice (evalPosCPUslice,
// networks/Word2Vec.scala:1007-1068).
template <int NR, bool SLICED>
__global__ void __launch_bounds__(kPosThreads)
    pos_eval_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                    const int *__restrict__ W, const int *__restrict__ LB,
                    const int *__restrict__ UB, const float *__restrict__ A,
                    const float *__restrict__ B, EvalScratch *scratch, float *retval, SliceMap sl) {
  constexpr int kChunk = EvalChunkOf<NR>::value;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = dim >> 2;
  const bool tail = lane + 32 * (NR - 1) < nvec;
  if (ncols_dev) ncols = *ncols_dev;
  const int per_block = (ncols + gridDim.x - 1) / gridDim.x;
  const int first = blockIdx.x * per_block;
  const int last = min(ncols, first + per_block);
  double acc = 0.0;

  // neighbouring positions go to the warps of one block: their windows overlap,
  // so most context rows are found in L1
  for (int t = first + warp; t < last; t += (int)(blockDim.x >> 5)) {
    const int wt = SLICED ? sl.local(W[t]) : W[t];
    if (wt < 0) continue;
    const int lbt = max(LB[t], -skip), ubt = min(UB[t], skip);
    Neighbour nb = look_at_neighbour(W, t, lbt, ubt, skip, ncols, lane);
    if (SLICED && nb.t_is_centre) {
      nb.word = sl.local(nb.word);
      nb.t_is_centre = nb.word >= 0;
    }
    unsigned todo = __ballot_sync(kFullMask, nb.t_is_centre);
    if (todo == 0) continue;
    PRow<NR> own;
    prow_load_lane(own, reinterpret_cast<const ulonglong2 *>(A + (int64_t)wt * dim) + lane, tail);
    auto take = [&](auto width) {
      constexpr int CH = decltype(width)::value;
      PRow<NR> rows[CH];
      float p[CH];
#pragma unroll
      for (int c = 0; c < CH; c++) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const int64_t w = __shfl_sync(kFullMask, nb.word, src);
        prow_load_lane(rows[c], reinterpret_cast<const ulonglong2 *>(B + w * dim) + lane, tail);
      }
#pragma unroll
      for (int c = 0; c < CH; c++) p[c] = prow_dot_partial(own, rows[c]);
      Spread<CH>::reduce(p, lane);
      // the lane that holds a pair's dot product scores it (networks/Word2Vec.scala:995)
      for_valid_totals<CH>(lane, [&](auto q) { acc += pair_score(sigmoid_guard(p[decltype(q)::value])); });
    };
    int cnt = __popc(todo);
    while (cnt > 0) {
      const int n = cnt > kChunk ? min(kChunk, (cnt + 1) >> 1) : cnt;
      cnt -= n;
      take_n<1, kChunk>(n, take);
    }
  }
  finish_eval_sum(acc, scratch, retval);
}

// Fallback for any dim / any alignment: rows are streamed from memory twice
// (dots first, then the updates), element by element.
__global__ void __launch_bounds__(kGenericThreads)
    pos_update_generic_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                              const int *__restrict__ W, const int *__restrict__ LB,
                              const int *__restrict__ UB, float *A, float *B, float lrate,
                              float vexp) {
  const int lane = threadIdx.x & 31;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;

  for (int i = gwarp; i < ncols; i += nwarps) {
    const int wc = W[i];
    if (wc < 0) continue;
    const int lb = max(LB[i], -skip), ub = min(UB[i], skip);
    const int wx = window_word(W, i, lb, ub, ncols, lane);
    const unsigned pairs = __ballot_sync(kFullMask, wx >= 0);
    if (pairs == 0) continue;
    const int sid = (lane == 31) ? wc : wx;
    const float sc = (sid >= 0) ? freq_scale(sid, vexp) : 0.f;
    const float sa = __shfl_sync(kFullMask, sc, 31);
    float *arow = A + (int64_t)wc * dim;

    float gmine = 0.f;  // lane src keeps lrate * (1 - sigmoid) of its pair
    for (unsigned todo = pairs; todo;) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const float *brow = B + (int64_t)__shfl_sync(kFullMask, wx, src) * dim;
      float p = 0.f;
      for (int c = lane; c < dim; c += 32) p = fmaf(arow[c], brow[c], p);
      p = warp_sum(p);
      if (lane == src) gmine = lrate * (1.0f - sigmoid_guard(p));
    }
    for (int c0 = 0; c0 < dim; c0 += 32) {
      const int c = c0 + lane;
      const float ac = (c < dim) ? arow[c] : 0.f;
      float dac = 0.f;
      for (unsigned todo = pairs; todo;) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        float *brow = B + (int64_t)__shfl_sync(kFullMask, wx, src) * dim;
        const float g = __shfl_sync(kFullMask, gmine, src);
        const float sb = __shfl_sync(kFullMask, sc, src);
        if (c < dim) {
          dac = fmaf(sa * g, brow[c], dac);
          atomicAdd(brow + c, sb * g * ac);
        }
      }
      if (c < dim) atomicAdd(arow + c, dac);
    }
  }
}

__global__ void __launch_bounds__(kGenericThreads)
    pos_eval_generic_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                            const int *__restrict__ W, const int *__restrict__ LB,
                            const int *__restrict__ UB, const float *__restrict__ A,
                            const float *__restrict__ B, EvalScratch *scratch, float *retval) {
  const int lane = threadIdx.x & 31;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  double acc = 0.0;
  for (int i = gwarp; i < ncols; i += nwarps) {
    const int wc = W[i];
    if (wc < 0) continue;
    const int lb = max(LB[i], -skip), ub = min(UB[i], skip);
    const int wx = window_word(W, i, lb, ub, ncols, lane);
    unsigned todo = __ballot_sync(kFullMask, wx >= 0);
    const float *arow = A + (int64_t)wc * dim;
    float mine = 0.f;
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const float *brow = B + (int64_t)__shfl_sync(kFullMask, wx, src) * dim;
      float p = 0.f;
      for (int c = lane; c < dim; c += 32) p = fmaf(arow[c], brow[c], p);
      p = warp_sum(p);
      if (lane == src) mine = p;
    }
    if (wx >= 0) acc += pair_score(sigmoid_guard(mine));
  }
  finish_eval_sum(acc, scratch, retval);
}

// ---------------------------------------------------------------------------
// Negative pairs
// ---------------------------------------------------------------------------

template <int NWA, int NWB, int NR>
__global__ void __launch_bounds__(kNegThreads)
    neg_update_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int nwords,
                      const int *__restrict__ WA, const int *__restrict__ WB, float *A, float *B,
                      float lrate, float vexp, HotRows hot) {
  using S = Spread<NWA * NWB>;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  int done = 0;

  for (int col = gwarp; col < ncols; col += nwarps) {
    const int myw = column_word<NWA, NWB>(WA, WB, col, nwords, lane);
    const float mysc = (myw >= 0) ? freq_scale(myw, vexp) : 0.f;

    Row<NR> a[NWA], b[NWB];
    int wa[NWA], wb[NWB];
#pragma unroll
    for (int j = 0; j < NWA; j++) {
      wa[j] = __shfl_sync(kFullMask, myw, j);
      if (wa[j] >= 0)
        row_load(a[j], A, wa[j], dim, nvec, lane);
      else
        row_zero(a[j]);
    }
#pragma unroll
    for (int k = 0; k < NWB; k++) {
      wb[k] = __shfl_sync(kFullMask, myw, NWA + k);
      if (wb[k] >= 0)
        row_load(b[k], B, wb[k], dim, nvec, lane);
      else
        row_zero(b[k]);
    }

    float p[NWA * NWB];
    column_dots<NWA, NWB, NR>(a, b, p, lane);
#pragma unroll
    for (int q = 0; q < S::FIN; q++) p[q] = -lrate * sigmoid_guard(p[q]);

    // every lane needs every pair's coefficient: fetch each from its owner
    float g[NWA * NWB];
    broadcast_totals<NWA * NWB>(p, g);

#pragma unroll
    for (int j = 0; j < NWA; j++) {
      const float sa = __shfl_sync(kFullMask, mysc, j);
      Row<NR> d;
      row_zero(d);
#pragma unroll
      for (int k = 0; k < NWB; k++) row_axpy(d, sa * g[j * NWB + k], b[k]);
      if (wa[j] >= 0)
        row_red_to(update_target(A, hot.shadowA, hot, wa[j], dim, gwarp), nvec, lane, d);
    }
#pragma unroll
    for (int k = 0; k < NWB; k++) {
      const float sb = __shfl_sync(kFullMask, mysc, NWA + k);
      Row<NR> d;
      row_zero(d);
#pragma unroll
      for (int j = 0; j < NWA; j++) row_axpy(d, sb * g[j * NWB + k], a[j]);
      if (wb[k] >= 0)
        row_red_to(update_target(B, hot.shadowB, hot, wb[k], dim, gwarp), nvec, lane, d);
    }
    if (hot.fold_every > 0 && (++done % hot.fold_every) == 0)
      fold_one_replica<NR>(hot, A, B, dim, nvec, lane, (unsigned)gwarp * 5u + (unsigned)(done / hot.fold_every));
  }
}

// ---------------------------------------------------------------------------
// Negative pairs, staged: the rows of a column are brought into shared memory
// by bulk asynchronous copies (one per row, completion counted on an mbarrier)
// one column ahead of the arithmetic, so a warp never waits for global memory
// in the middle of a column.  Each warp is its own pipeline with one stage.
//
// Shared memory per warp: 256-byte header (mbarrier, word ids of the staged
// column) + one stage of (NWA + NWB) rows.
// ---------------------------------------------------------------------------
constexpr int kStagedHeader = 256;
constexpr int kWaitPolls = 1 << 20;  // polls of a stage's barrier before giving up


// The smaller side of the column (NX rows) is held in registers, the larger
// side (NY rows) is read from the stage twice: for the dot products and for the
// deltas of the held side, by which time the held rows' registers are free to
// carry them; its own deltas need the held rows only.
// The stage is refilled with the warp's next column when the column is done.
template <int NWA, int NWB, int NR>
struct StagedShape {
  static constexpr int held = (NWB <= NWA) ? NWB : NWA;
  // threads per block the kernel is compiled for: 16 warps (128 registers per
  // thread) when the held rows and the pair coefficients are few, else 12 (168)
  static constexpr int max_threads = (held * NR <= 15 && NWA * NWB <= 25) ? 512 : 384;
};

__host__ __device__ inline size_t staged_warp_bytes(int nrows_per_col, int dim, int stages) {
  return kStagedHeader + (size_t)stages * nrows_per_col * dim * sizeof(float);
}

// EVAL = true turns the same pipeline into the scoring kernel (the name keeps
// "update" for both): no updates, the lane that holds a pair's dot product adds
// log(max(1 - sigmoid, 1e-20)).
// SLICED: WA / WB hold global ids and A / B the rows of one vocabulary slice (SliceMap).  A word
// without a row here acts as a masked one; head-head pairs contribute nothing unless do_head > 1
// and head rows are written only when do_head > 0 (word2vecNegSlice, BIDMach_CPUMACH.c:267-366);
// the score counts the pairs whose two words both have a row here (evalNegCPUslice,
// networks/Word2Vec.scala:1134-1200).
template <int NWA, int NWB, int NR, bool EVAL, bool SLICED>
__global__ void __launch_bounds__((StagedShape<NWA, NWB, NR>::max_threads), 1)
    neg_update_staged_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int nwords,
                      const int *__restrict__ WA, const int *__restrict__ WB, float *A, float *B,
                      float lrate, float vexp, HotRows hot, EvalScratch *scratch, float *retval,
                      int *fault, SliceMap sl) {
  using S = Spread<NWA * NWB>;
  constexpr int NROWS = NWA + NWB;
  constexpr int NST = 1;
  constexpr bool HOLD_B = (NWB <= NWA);     // which side stays in registers when streaming
  constexpr int NX = HOLD_B ? NWB : NWA;    // held rows
  constexpr int NY = HOLD_B ? NWA : NWB;    // other rows
  constexpr int XOFF = HOLD_B ? NWA : 0;    // first held row inside a stage
  constexpr int YOFF = HOLD_B ? 0 : NWA;    // first other row inside a stage
  extern __shared__ __align__(128) unsigned char staged_smem[];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = dim >> 2;
  const unsigned rowbytes = (unsigned)dim * 4u;
  const size_t stage_bytes = (size_t)NROWS * rowbytes;
  unsigned char *mine = staged_smem + (size_t)warp * staged_warp_bytes(NROWS, dim, NST);
  u64 *bars = reinterpret_cast<u64 *>(mine);            // [NST]
  int *ids = reinterpret_cast<int *>(mine + 64);        // [NST][16]
  unsigned char *stages = mine + kStagedHeader;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  float *const MX = HOLD_B ? B : A, *const MY = HOLD_B ? A : B;
  float *const SX = HOLD_B ? hot.shadowB : hot.shadowA, *const SY = HOLD_B ? hot.shadowA : hot.shadowB;

  if (lane == 0)
    for (int st = 0; st < NST; st++) mbar_init(&bars[st], 1);
  mbar_init_fence();
  __syncwarp();

  const int mycols = (gwarp < ncols) ? (ncols - gwarp + nwarps - 1) / nwarps : 0;
  double acc = 0.0;  // EVAL: this lane's share of the score
  const bool tail = lane + 32 * (NR - 1) < nvec;
  const int fold_every = fold_period(hot, lrate, (float)NWB);
  int until_fold = fold_every;
  unsigned fold_turn = (unsigned)gwarp * 5u;

  // Starts the copies of a column (word ids in `w`, one per lane) into stage `st`.
  auto fill = [&](int st, int w) {
    if (lane < 16) ids[st * 16 + lane] = w;
    async_proxy_fence();  // earlier reads of this stage come before the new writes
    const bool want = (lane < NROWS) && (w >= 0);
    const unsigned wanted = __ballot_sync(kFullMask, want);
    if (lane == 0) mbar_arrive_expect_tx(&bars[st], (unsigned)__popc(wanted) * rowbytes);
    __syncwarp();
    if (want) {
      const float *src = (lane < NWA ? A : B) + (int64_t)w * dim;
      bulk_load_row(stages + st * stage_bytes + (size_t)lane * rowbytes, src, rowbytes, &bars[st]);
    }
  };
  auto ids_of = [&](int i) {
    int w = column_word<NWA, NWB>(WA, WB, gwarp + (int64_t)i * nwarps, nwords, lane);
    if (SLICED) {
      w = sl.local(w);
      // a column without a single pair that counts is dropped whole, before any of its rows is
      // fetched: for the update, one without a word of this slice's own when head-head pairs are
      // left out; for either kind, one whose A side or B side has no row here at all
      const unsigned have = __ballot_sync(kFullMask, w >= 0);
      const unsigned own = __ballot_sync(kFullMask, w >= sl.nhead);
      const bool none = (have & ((1u << NWA) - 1u)) == 0u || (have >> NWA) == 0u ||
                        (!EVAL && sl.skips_head_pairs() && own == 0u);
      if (none) w = -1;
    }
    return w;
  };
  // a row that takes part may still be closed to writes (head rows of a slice with do_head 0)
  auto writable = [&](int w) { return w >= 0 && !(SLICED && sl.freezes_head() && w < sl.nhead); };

  if (mycols > 0) fill(0, ids_of(0));
  int ahead = (mycols > 1) ? ids_of(1) : -1;  // word ids of the next column to fill

  for (int i = 0; i < mycols; i++) {
    const int st = i % NST;
    if (!__all_sync(kFullMask, mbar_wait_bounded(&bars[st], (unsigned)(i / NST) & 1u, kWaitPolls))) {
      // the copies never completed within the limit (this warp has no other
      // copy in flight): report and stop, the whole warp together
      if (lane == 0 && fault) {
        *reinterpret_cast<volatile int *>(fault) = 1;
        __threadfence_system();
      }
      break;
    }
    const int myw = (lane < 16) ? ids[st * 16 + lane] : -1;
    const float mysc = (myw >= 0) ? freq_scale(SLICED ? sl.global(myw) : myw, vexp) : 0.f;
    const ulonglong2 *stage = reinterpret_cast<const ulonglong2 *>(stages + st * stage_bytes) + lane;
    auto staged_row = [&](int r) {  // this lane's first vector of row r of the stage
      return reinterpret_cast<const ulonglong2 *>(reinterpret_cast<const unsigned char *>(stage) +
                                                  (size_t)r * rowbytes);
    };

    auto refill = [&]() {
      if (i + 1 < mycols) {
        fill(0, ahead);
        if (i + 2 < mycols) ahead = ids_of(i + 2);
      }
    };
    if (SLICED && !__any_sync(kFullMask, myw >= 0)) {   // a dropped column: nothing was fetched
      __syncwarp();
      refill();
      continue;
    }
    // CHECKED = false: every word of the column is present (the usual case), so
    // no row needs a test; CHECKED = true: masked words act as zero rows and
    // receive no update.
    auto column = [&](auto checked_t) {
      constexpr bool CHECKED = decltype(checked_t)::value;
      PRow<NR> X[NX];
      int wx[NX];
#pragma unroll
      for (int x = 0; x < NX; x++) {
        wx[x] = __shfl_sync(kFullMask, myw, XOFF + x);
        if (!CHECKED || wx[x] >= 0)
          prow_load_lane(X[x], staged_row(XOFF + x), tail);
        else
          prow_zero(X[x]);
      }
      float p[NWA * NWB];
      float sx[NX];
#pragma unroll
      for (int x = 0; x < NX; x++) sx[x] = __shfl_sync(kFullMask, mysc, XOFF + x);
#pragma unroll
      for (int y = 0; y < NY; y++) {
        PRow<NR> Y;
        if (!CHECKED || __shfl_sync(kFullMask, myw, YOFF + y) >= 0)
          prow_load_lane(Y, staged_row(YOFF + y), tail);
        else
          prow_zero(Y);
#pragma unroll
        for (int x = 0; x < NX; x++)
          p[HOLD_B ? (y * NWB + x) : (x * NWB + y)] = prow_dot_partial(X[x], Y);
      }
      if constexpr (EVAL) {
        __syncwarp();  // scoring needs the stage no longer: the next column's copies start now
        refill();
      }
      S::reduce(p, lane);
      if constexpr (EVAL) {
        for_valid_totals<NWA * NWB>(
            lane, [&](auto q) { acc += pair_score(1.0f - sigmoid_guard(p[decltype(q)::value])); });
        if constexpr (SLICED) {
          // a pair with a word that has no row here was scored as a pair with a zero row,
          // log(1/2): take those out again, the slice's score counts only its own pairs
          const unsigned have = __ballot_sync(kFullMask, myw >= 0);
          const int na = __popc(have & ((1u << NWA) - 1u)), nb = __popc(have >> NWA);
          if (lane == 0) acc -= (double)(NWA * NWB - na * nb) * pair_score(0.5f);
        }
      } else {
#pragma unroll
        for (int q = 0; q < S::FIN; q++) p[q] = -lrate * sigmoid_guard(p[q]);
        float g[NWA * NWB];
        broadcast_totals<NWA * NWB>(p, g);
        unsigned live_a = (1u << NWA) - 1u, live_b = (1u << NWB) - 1u;   // rows with a pair that counts
        if constexpr (SLICED) {
          // a pair counts when both words have a row here and it is not a head-head pair that the
          // slice leaves out; the others get a zero coefficient, and a row none of whose pairs
          // counts is not written at all (most rows of a slice's minibatch, which would otherwise
          // cost an atomic row addition of zeros each)
          const unsigned have = __ballot_sync(kFullMask, myw >= 0);
          const unsigned head = sl.skips_head_pairs() ? __ballot_sync(kFullMask, myw >= 0 && myw < sl.nhead) : 0u;
          live_a = live_b = 0u;
#pragma unroll
          for (int j = 0; j < NWA; j++)
#pragma unroll
            for (int k = 0; k < NWB; k++) {
              const bool both = ((have >> j) & 1u) && ((have >> (NWA + k)) & 1u);
              const bool hh = ((head >> j) & 1u) && ((head >> (NWA + k)) & 1u);
              if (both && !hh) {
                live_a |= 1u << j;
                live_b |= 1u << k;
              } else {
                g[j * NWB + k] = 0.f;
              }
            }
        }
        auto row_live = [&](bool is_a, int idx) { return ((is_a ? live_a : live_b) >> idx) & 1u; };
        // rows of the streamed side: their deltas need the held rows only
#pragma unroll
        for (int y = 0; y < NY; y++) {
          const int wy = __shfl_sync(kFullMask, myw, YOFF + y);
          const float sy = __shfl_sync(kFullMask, mysc, YOFF + y);
          PRow<NR> dY;
          prow_scale(dY, sy * g[HOLD_B ? (y * NWB + 0) : (0 * NWB + y)], X[0]);
#pragma unroll
          for (int x = 1; x < NX; x++)
            prow_axpy(dY, sy * g[HOLD_B ? (y * NWB + x) : (x * NWB + y)], X[x]);
          if ((!CHECKED || writable(wy)) && (!SLICED || row_live(HOLD_B, y)))
            prow_red_lane(update_target(MY, SY, hot, wy, dim, gwarp) + 4 * lane, tail, dY);
        }
        // rows of the held side: the held rows themselves are dead by now, their
        // registers carry the deltas while the other side streams by once more
        if constexpr (CHECKED) {
#pragma unroll
          for (int x = 0; x < NX; x++) prow_zero(X[x]);
        }
#pragma unroll
        for (int y = 0; y < NY; y++) {
          if (CHECKED && __shfl_sync(kFullMask, myw, YOFF + y) < 0) continue;
          PRow<NR> Y;
          prow_load_lane(Y, staged_row(YOFF + y), tail);
#pragma unroll
          for (int x = 0; x < NX; x++) {
            const float c = sx[x] * g[HOLD_B ? (y * NWB + x) : (x * NWB + y)];
            if (!CHECKED && y == 0)
              prow_scale(X[x], c, Y);
            else
              prow_axpy(X[x], c, Y);
          }
        }
#pragma unroll
        for (int x = 0; x < NX; x++)
          if ((!CHECKED || writable(wx[x])) && (!SLICED || row_live(!HOLD_B, x)))
            prow_red_lane(update_target(MX, SX, hot, wx[x], dim, gwarp) + 4 * lane, tail, X[x]);
      }
    };
    if (!SLICED && __all_sync(kFullMask, lane >= NROWS || myw >= 0))
      column(std::false_type());
    else
      column(std::true_type());
    if constexpr (!EVAL) {
      __syncwarp();  // every lane is done with this stage: start the copies of the next column
      refill();
    }
    if (!EVAL && fold_every > 0 && --until_fold == 0) {
      until_fold = fold_every;
      fold_one_replica<NR>(hot, A, B, dim, nvec, lane, fold_turn++);
    }
  }
  if constexpr (EVAL) finish_eval_sum(acc, scratch, retval);
}

// Scoring of the negative columns: the smaller side of a column is held in
// registers, the rows of the other side stream through once, straight from
// global memory (nothing is written, so there is nothing to stage around).
template <int NWA, int NWB, int NR>
struct NegEvalShape {
  static constexpr int held = (NWB <= NWA) ? NWB : NWA;
  static constexpr int blocks = (held * NR <= 15) ? 4 : 2;  // resident blocks of kNegThreads per SM
};

template <int NWA, int NWB, int NR>
__global__ void __launch_bounds__(kNegThreads, (NegEvalShape<NWA, NWB, NR>::blocks))
    neg_eval_kernel(int dim, int ncols, const int *__restrict__ ncols_dev,
                    const int *__restrict__ WA, const int *__restrict__ WB,
                    const float *__restrict__ A, const float *__restrict__ B,
                    EvalScratch *scratch, float *retval, int wa_stride, int wb_stride) {
  // wa_stride / wb_stride: words per column in WA / WB (NWA / NWB, or more when
  // this launch scores one half of a wider column)
  using S = Spread<NWA * NWB>;
  constexpr bool HOLD_B = (NWB <= NWA);
  constexpr int NX = HOLD_B ? NWB : NWA, NY = HOLD_B ? NWA : NWB;
  constexpr int XOFF = HOLD_B ? NWA : 0, YOFF = HOLD_B ? 0 : NWA;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
  const bool tail = lane + 32 * (NR - 1) < nvec;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  const float *const MX = HOLD_B ? B : A, *const MY = HOLD_B ? A : B;
  double acc = 0.0;

  for (int col = gwarp; col < ncols; col += nwarps) {
    int myw = 0;
    if (lane < NWA)
      myw = WA[(int64_t)col * wa_stride + lane];
    else if (lane < NWA + NWB)
      myw = WB[(int64_t)col * wb_stride + (lane - NWA)];
    PRow<NR> X[NX];
#pragma unroll
    for (int x = 0; x < NX; x++) {
      const int64_t w = __shfl_sync(kFullMask, myw, XOFF + x);
      if (w >= 0)   // a masked id (-1) scores as a zero row, as in the staged kernel
        prow_load_lane(X[x], reinterpret_cast<const ulonglong2 *>(MX + w * dim) + lane, tail);
      else
        prow_zero(X[x]);
    }
    float p[NWA * NWB];
#pragma unroll
    for (int y = 0; y < NY; y++) {
      const int64_t w = __shfl_sync(kFullMask, myw, YOFF + y);
      PRow<NR> Y;
      if (w >= 0)
        prow_load_lane(Y, reinterpret_cast<const ulonglong2 *>(MY + w * dim) + lane, tail);
      else
        prow_zero(Y);
#pragma unroll
      for (int x = 0; x < NX; x++)
        p[HOLD_B ? (y * NWB + x) : (x * NWB + y)] = prow_dot_partial(X[x], Y);
    }
    S::reduce(p, lane);
    for_valid_totals<NWA * NWB>(
        lane, [&](auto q) { acc += pair_score(1.0f - sigmoid_guard(p[decltype(q)::value])); });
  }
  finish_eval_sum(acc, scratch, retval);
}

// Fallback for any dim / alignment, two passes over the rows of a column.
template <int NWA, int NWB, bool EVAL>
__global__ void __launch_bounds__(kGenericThreads)
    neg_generic_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int nwords,
                       const int *__restrict__ WA, const int *__restrict__ WB, float *A, float *B,
                       float lrate, float vexp, EvalScratch *scratch, float *retval) {
  using S = Spread<NWA * NWB>;
  const int lane = threadIdx.x & 31;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  double acc = 0.0;

  for (int col = gwarp; col < ncols; col += nwarps) {
    const int myw = column_word<NWA, NWB>(WA, WB, col, nwords, lane);
    const float mysc = (myw >= 0 && !EVAL) ? freq_scale(myw, vexp) : 0.f;
    int wa[NWA], wb[NWB];
#pragma unroll
    for (int j = 0; j < NWA; j++) wa[j] = __shfl_sync(kFullMask, myw, j);
#pragma unroll
    for (int k = 0; k < NWB; k++) wb[k] = __shfl_sync(kFullMask, myw, NWA + k);

    float p[NWA * NWB];
#pragma unroll
    for (int idx = 0; idx < NWA * NWB; idx++) p[idx] = 0.f;
    for (int c = lane; c < dim; c += 32) {
      float av[NWA], bv[NWB];
#pragma unroll
      for (int j = 0; j < NWA; j++) av[j] = (wa[j] >= 0) ? A[(int64_t)wa[j] * dim + c] : 0.f;
#pragma unroll
      for (int k = 0; k < NWB; k++) bv[k] = (wb[k] >= 0) ? B[(int64_t)wb[k] * dim + c] : 0.f;
#pragma unroll
      for (int j = 0; j < NWA; j++)
#pragma unroll
        for (int k = 0; k < NWB; k++) p[j * NWB + k] = fmaf(av[j], bv[k], p[j * NWB + k]);
    }
    S::reduce(p, lane);

    if constexpr (EVAL) {
      for_valid_totals<NWA * NWB>(
          lane, [&](auto q) { acc += pair_score(1.0f - sigmoid_guard(p[decltype(q)::value])); });
    } else {
#pragma unroll
    for (int q = 0; q < S::FIN; q++) p[q] = -lrate * sigmoid_guard(p[q]);
    float g[NWA * NWB];
    broadcast_totals<NWA * NWB>(p, g);
    float sa[NWA], sb[NWB];
#pragma unroll
    for (int j = 0; j < NWA; j++) sa[j] = __shfl_sync(kFullMask, mysc, j);
#pragma unroll
    for (int k = 0; k < NWB; k++) sb[k] = __shfl_sync(kFullMask, mysc, NWA + k);

    for (int c = lane; c < dim; c += 32) {
      float av[NWA], bv[NWB];
#pragma unroll
      for (int j = 0; j < NWA; j++) av[j] = (wa[j] >= 0) ? A[(int64_t)wa[j] * dim + c] : 0.f;
#pragma unroll
      for (int k = 0; k < NWB; k++) bv[k] = (wb[k] >= 0) ? B[(int64_t)wb[k] * dim + c] : 0.f;
#pragma unroll
      for (int j = 0; j < NWA; j++) {
        float d = 0.f;
#pragma unroll
        for (int k = 0; k < NWB; k++) d = fmaf(sa[j] * g[j * NWB + k], bv[k], d);
        if (wa[j] >= 0) atomicAdd(A + (int64_t)wa[j] * dim + c, d);
      }
#pragma unroll
      for (int k = 0; k < NWB; k++) {
        float d = 0.f;
#pragma unroll
        for (int j = 0; j < NWA; j++) d = fmaf(sb[k] * g[j * NWB + k], av[j], d);
        if (wb[k] >= 0) atomicAdd(B + (int64_t)wb[k] * dim + c, d);
      }
    }
    }
  }
  if (EVAL) finish_eval_sum(acc, scratch, retval);
}

// ---------------------------------------------------------------------------
// Host side: device facts, scratch, dispatch
// ---------------------------------------------------------------------------

static std::atomic<long long> g_launches{0};

long long launch_count() { return g_launches.load(); }
void count_launch(int n) { g_launches.fetch_add(n); }

// SMs the calling thread's launches leave free (see SmReserve).
static thread_local int t_sm_reserve = 0;

SmReserve::SmReserve(int sms) : previous(t_sm_reserve) { t_sm_reserve = sms > 0 ? sms : 0; }
SmReserve::~SmReserve() { t_sm_reserve = previous; }

int device_sm_count() {
  thread_local int cached_dev = -1, cached_sms = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    cached_dev = dev;
    cached_sms = sms;
  }
  return std::max(1, cached_sms - t_sm_reserve);
}

// Replica rows for the hot ids: 64 rows per level and matrix, sized for the
// widest supported row.  One buffer per (host thread, device) for the
// synchronous entry points; a minibatch context owns its own.
constexpr int kHotMaxLevels = 6;
constexpr int kHotMaxDim = 1280;

int hot_levels_default() {
  static int levels = [] {
    const char *e = getenv("W2V_HOT_LEVELS");
    int v = e ? atoi(e) : 4;
    return v < 0 ? 0 : (v > kHotMaxLevels ? kHotMaxLevels : v);
  }();
  return levels;
}

size_t hot_rows_bytes() { return sizeof(float) * 2 * 64 * kHotMaxLevels * (size_t)kHotMaxDim; }

HotRows hot_rows_at(float *buffer, int levels) {
  HotRows h;
  h.shadowA = buffer;
  h.shadowB = buffer ? buffer + (size_t)64 * kHotMaxLevels * kHotMaxDim : nullptr;
  static const int rmax = [] {
    const char *e = getenv("W2V_HOT_REPS");
    int v = e ? atoi(e) : 16;
    int p2 = 2;
    while (p2 * 2 <= v && p2 < 64) p2 *= 2;
    return p2;
  }();
  h.rmax = rmax;
  while (levels > 0 && (rmax >> (levels - 1)) < 1) levels--;  // every level needs at least one replica
  h.limit = (buffer && levels > 0) ? (1 << levels) : 0;
  // a warp folds one replica row every `fold_every` columns (negative kernel) or
  // every 2 * fold_every positions (positive kernel); 0 leaves everything to the
  // fold kernel that follows the update kernel.  64 is a compromise: a period of 16 makes the
  // first minibatches of a run (model still near its start, every update of a frequent word
  // matters) learn as fast as plain atomics do -- held-out gain after six 1M-token subsampled
  // minibatches at vocab 1M: 88 % of the sequential CPU kernels' with 16, 90 % with plain
  // atomics, 70 % with 64, the gap closing as training goes on -- but costs 6 % of the
  // throughput on that text and 17 % on dense text (W2V_FOLD_EVERY selects it).
  static const int every = [] {
    const char *e = getenv("W2V_FOLD_EVERY");
    return e ? atoi(e) : 64;
  }();
  h.fold_every = h.limit > 1 ? every : 0;
  h.stats = nullptr;
  return h;
}

// Pool of launcher scratch sets, one list per device.
namespace {
constexpr int kPoolMaxDev = 64;
std::mutex g_pool_mutex;
LaunchScratch *g_pool_free[kPoolMaxDev] = {nullptr};
constexpr size_t kScratchTail = 256;  // bytes after the replica rows: stats at +0, accumulator at +64
}  // namespace

int acquire_launch_scratch(LaunchScratch **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kPoolMaxDev) return (int)cudaErrorInvalidDevice;
  {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (LaunchScratch *s = g_pool_free[dev]) {
      g_pool_free[dev] = s->next;
      s->next = nullptr;
      *out = s;
      return 0;
    }
  }
  // every set on this device is in use by another thread's call: make one more
  const size_t hot_bytes = hot_levels_default() > 0 ? hot_rows_bytes() : 0;
  unsigned char *p = nullptr;
  e = cudaMalloc(&p, hot_bytes + kScratchTail);
  if (e != cudaSuccess) return (int)e;
  int *fault = nullptr;
  e = cudaHostAlloc(&fault, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) {
    *fault = 0;
    e = cudaMemsetAsync(p, 0, hot_bytes + kScratchTail, cudaStreamPerThread);
  }
  if (e != cudaSuccess) {
    cudaFree(p);
    if (fault) cudaFreeHost(fault);
    return (int)e;
  }
  LaunchScratch *s = new LaunchScratch();
  s->hot_buf = hot_bytes ? reinterpret_cast<float *>(p) : nullptr;
  s->stats = reinterpret_cast<int *>(p + hot_bytes);
  s->eval = reinterpret_cast<EvalScratch *>(p + hot_bytes + 64);
  s->fault = fault;
  s->device = dev;
  s->next = nullptr;
  *out = s;
  return 0;
}

void release_launch_scratch(LaunchScratch *s) {
  if (!s) return;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  s->next = g_pool_free[s->device];
  g_pool_free[s->device] = s;
}

__global__ void hot_share_kernel(const int *__restrict__ ids, int64_t n, int nwords,
                                 int *__restrict__ stats) {
  int valid = 0, zeros = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int w = ids[i];
    valid += (w >= 0 && w < nwords);
    zeros += (w == 0);
  }
  __shared__ int part[2];
  if (threadIdx.x == 0) part[0] = part[1] = 0;
  __syncthreads();
  valid = __reduce_add_sync(kFullMask, valid);
  zeros = __reduce_add_sync(kFullMask, zeros);
  if ((threadIdx.x & 31) == 0) {
    if (valid) atomicAdd(&part[0], valid);
    if (zeros) atomicAdd(&part[1], zeros);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (part[0]) atomicAdd(&stats[0], part[0]);
    if (part[1]) atomicAdd(&stats[1], part[1]);
  }
}

int count_hot_share_async(const int *ids, int64_t n, int nwords, int *stats, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(stats, 0, 2 * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  if (n <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)std::min<int64_t>((n + threads * 8 - 1) / (threads * 8), (int64_t)device_sm_count() * 4);
  hot_share_kernel<<<std::max(1, blocks), threads, 0, stream>>>(ids, n, nwords, stats);
  count_launch(1);
  return (int)cudaGetLastError();
}

static void fold_hot_rows(int dim, const HotRows &hot, float *A, float *B, cudaStream_t stream) {
  if (hot.limit <= 1) return;
  hot_fold_kernel<<<dim3(hot.limit - 1, 2), 128, 0, stream>>>(dim, hot, A, B);
  count_launch(1);
}

static inline bool vector_ok(int dim, const void *A, const void *B) {
  return dim > 0 && (dim & 3) == 0 && dim <= 1280 && ((uintptr_t)A & 15) == 0 &&
         ((uintptr_t)B & 15) == 0;
}

static inline int grid_for(int work_items, int threads, int blocks_per_sm) {
  int warps_per_block = threads / 32;
  long long need = ((long long)work_items + warps_per_block - 1) / warps_per_block;
  long long cap = (long long)device_sm_count() * blocks_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

#define W2V_NR_SWITCH(NRV, CALL)        \
  switch (NRV) {                        \
    case 1: { constexpr int NR = 1; CALL; } break;   \
    case 2: { constexpr int NR = 2; CALL; } break;   \
    case 3: { constexpr int NR = 3; CALL; } break;   \
    case 4: { constexpr int NR = 4; CALL; } break;   \
    case 5: { constexpr int NR = 5; CALL; } break;   \
    case 6: { constexpr int NR = 6; CALL; } break;   \
    case 7: { constexpr int NR = 7; CALL; } break;   \
    case 8: { constexpr int NR = 8; CALL; } break;   \
    case 9: { constexpr int NR = 9; CALL; } break;   \
    default: { constexpr int NR = 10; CALL; } break; \
  }

template <int NR, bool SLICED>
static cudaError_t launch_pos_update(int grid, size_t smem, cudaStream_t stream, int dim, int ncols,
                                     const int *ncols_dev, int skip, const int *W, const int *LB,
                                     const int *UB, float *A, float *B, float lrate, float vexp,
                                     const HotRows &hot, const SliceMap &sl, int yield_dense) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(pos_update_kernel<NR, SLICED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  pos_update_kernel<NR, SLICED><<<grid, kPosThreads, smem, stream>>>(dim, ncols, ncols_dev, skip, W, LB,
                                                                     UB, A, B, lrate, vexp, hot, sl, yield_dense);
  return cudaSuccess;
}

template <int NR>
static cudaError_t launch_pos_pair(int grid, size_t smem, cudaStream_t stream, int dim, int ncols,
                                   const int *ncols_dev, int skip, const int *W, const int *LB, const int *UB,
                                   float *A, float *B, float lrate, float vexp, const HotRows &hot) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(pos_update_pair_kernel<NR>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  pos_update_pair_kernel<NR><<<grid, kPosThreads, smem, stream>>>(dim, ncols, ncols_dev, skip, W, LB, UB, A, B,
                                                                  lrate, vexp, hot);
  return cudaSuccess;
}

// Launch shape of the positive update for rows of `dim` floats and window
// half-width `skip`: shared memory per block, or 0 when the ring does not fit.
static size_t pos_ring_bytes(int dim, int skip) {
  return (size_t)(kPosThreads / 32) * (2 * skip + 1) * (size_t)dim * sizeof(float);
}

int pos_update_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W,
                     const int *LB, const int *UB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, const SliceMap &slice, cudaStream_t stream) {
  if (ncols <= 0) return 0;
  if (skip < 1 || skip > 15) return 1;
  const size_t smem = pos_ring_bytes(dim, skip);
  const bool sliced = !slice.whole();
  if (sliced && !(vector_ok(dim, A, B) && smem <= 227 * 1024)) {
    printf("word2vecPosSlice needs rows of a multiple of 4 floats, 16-byte aligned matrices (dim %d)\n", dim);
    return 1;
  }
  if (vector_ok(dim, A, B) && smem <= 227 * 1024) {
    const int nr = (dim / 4 + 31) / 32;
    const int resident = (int)std::min<size_t>(4, (227 * 1024) / smem);
    // enough warps to fill the GPU, but stretches of at least ~64 positions so
    // that the window edges between stretches stay a small share of the work
    int grid = device_sm_count() * resident;
    const int max_grid = std::max(1, ncols / (64 * (kPosThreads / 32)));
    grid = std::max(1, std::min(grid, max_grid));
    cudaError_t e = cudaSuccess;
    // two centres at a time for dense text, where three blocks of its ring fit an SM: launched
    // beside the kernel for one centre at a time, the count of valid words on the device decides
    // which of the two goes on (pos_text_is_dense)
    const size_t smem_pair = (size_t)(kPosThreads / 32) * (2 * skip + 2) * (size_t)dim * sizeof(float);
    const bool pair_too = !sliced && nr <= 4 && hot.stats != nullptr && 3 * (smem_pair + 1024) <= 228 * 1024;
    if (sliced) {
      W2V_NR_SWITCH(nr, (e = launch_pos_update<NR, true>(grid, smem, stream, dim, ncols, ncols_dev, skip, W,
                                                         LB, UB, A, B, lrate, vexp, hot, slice, 0)));
    } else {
      W2V_NR_SWITCH(nr, (e = launch_pos_update<NR, false>(grid, smem, stream, dim, ncols, ncols_dev, skip, W,
                                                          LB, UB, A, B, lrate, vexp, hot, slice, pair_too ? 1 : 0)));
    }
    if (e == cudaSuccess && pair_too) {
      const int grid2 = std::max(1, std::min(device_sm_count() * 3, max_grid));
      switch (nr) {
        case 1: e = launch_pos_pair<1>(grid2, smem_pair, stream, dim, ncols, ncols_dev, skip, W, LB, UB, A, B, lrate, vexp, hot); break;
        case 2: e = launch_pos_pair<2>(grid2, smem_pair, stream, dim, ncols, ncols_dev, skip, W, LB, UB, A, B, lrate, vexp, hot); break;
        case 3: e = launch_pos_pair<3>(grid2, smem_pair, stream, dim, ncols, ncols_dev, skip, W, LB, UB, A, B, lrate, vexp, hot); break;
        default: e = launch_pos_pair<4>(grid2, smem_pair, stream, dim, ncols, ncols_dev, skip, W, LB, UB, A, B, lrate, vexp, hot); break;
      }
      count_launch(1);
    }
    if (e != cudaSuccess) return (int)e;
    fold_hot_rows(dim, hot, A, B, stream);
  } else {
    const int grid = grid_for(ncols, kGenericThreads, 16);
    pos_update_generic_kernel<<<grid, kGenericThreads, 0, stream>>>(dim, ncols, ncols_dev, skip, W,
                                                                    LB, UB, A, B, lrate, vexp);
  }
  count_launch(1);
  return (int)cudaGetLastError();
}

int pos_eval_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W, const int *LB,
                   const int *UB, const float *A, const float *B, float *retval,
                   EvalScratch *scratch, const SliceMap &slice, cudaStream_t stream) {
  if (ncols <= 0) return 0;
  if (skip < 1 || skip > 15) return 1;
  const bool sliced = !slice.whole();
  if (sliced && !vector_ok(dim, A, B)) {
    printf("word2vecEvalPosSlice needs rows of a multiple of 4 floats, 16-byte aligned matrices (dim %d)\n", dim);
    return 1;
  }
  if (vector_ok(dim, A, B)) {
    const int nr = (dim / 4 + 31) / 32;
    const int grid = grid_for(ncols, kPosThreads, 8);
    if (sliced) {
      W2V_NR_SWITCH(nr, (pos_eval_kernel<NR, true><<<grid, kPosThreads, 0, stream>>>(
                            dim, ncols, ncols_dev, skip, W, LB, UB, A, B, scratch, retval, slice)));
    } else {
      W2V_NR_SWITCH(nr, (pos_eval_kernel<NR, false><<<grid, kPosThreads, 0, stream>>>(
                            dim, ncols, ncols_dev, skip, W, LB, UB, A, B, scratch, retval, slice)));
    }
  } else {
    const int grid = grid_for(ncols, kGenericThreads, 16);
    pos_eval_generic_kernel<<<grid, kGenericThreads, 0, stream>>>(
        dim, ncols, ncols_dev, skip, W, LB, UB, A, B, scratch, retval);
  }
  count_launch(1);
  return (int)cudaGetLastError();
}

// blocks per SM the negative scoring grid is cut into (four are resident at a time;
// more and shorter blocks even out the tail: measured 1.78 / 1.74 / 1.71 ms at 4 / 8 / 16)
constexpr int kNegEvalGridBlocks = 16;

static bool neg_staged_enabled() {
  static bool on = [] {
    const char *e = getenv("W2V_NEG_IMPL");
    return !(e && e[0] == 'r');  // "reg" selects the register-resident kernel
  }();
  return on;
}

template <int NWA, int NWB, int NR, bool EVAL, bool SLICED>
static cudaError_t launch_neg_staged(int grid, int warps, size_t smem, cudaStream_t stream, int dim,
                                     int ncols, const int *ncols_dev, int nwords, const int *WA,
                                     const int *WB, float *A, float *B, float lrate, float vexp,
                                     const HotRows &hot, EvalScratch *scratch, float *retval,
                                     int *fault, const SliceMap &sl) {
  // never more threads than the kernel was compiled for
  constexpr int kMaxWarps = StagedShape<NWA, NWB, NR>::max_threads / 32;
  if (warps > kMaxWarps) {
    warps = kMaxWarps;
    smem = staged_warp_bytes(NWA + NWB, dim, 1) * warps;
  }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(neg_update_staged_kernel<NWA, NWB, NR, EVAL, SLICED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  neg_update_staged_kernel<NWA, NWB, NR, EVAL, SLICED><<<grid, warps * 32, smem, stream>>>(
      dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot, scratch, retval, fault, sl);
  return cudaSuccess;
}

template <int NWA, int NWB, int NR>
static cudaError_t launch_neg_staged_any(bool eval, int grid, int warps, size_t smem,
                                         cudaStream_t stream, int dim, int ncols,
                                         const int *ncols_dev, int nwords, const int *WA,
                                         const int *WB, float *A, float *B, float lrate, float vexp,
                                         const HotRows &hot, EvalScratch *scratch, float *retval,
                                         int *fault, const SliceMap &sl) {
#define W2V_STAGED(EV, SL)                                                                                  \
  launch_neg_staged<NWA, NWB, NR, EV, SL>(grid, warps, smem, stream, dim, ncols, ncols_dev, nwords, WA, WB, \
                                          A, B, lrate, vexp, hot, scratch, retval, fault, sl)
  if (sl.whole()) return eval ? W2V_STAGED(true, false) : W2V_STAGED(false, false);
  return eval ? W2V_STAGED(true, true) : W2V_STAGED(false, true);
#undef W2V_STAGED
}

template <int NWA, int NWB>
static int neg_dispatch(bool eval, int dim, int ncols, const int *ncols_dev, int nwords,
                        const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                        float *retval, const HotRows &hot, EvalScratch *scratch, int *fault,
                        const SliceMap &sl, cudaStream_t stream) {
  const int nr = (dim / 4 + 31) / 32;
  // rows of a column live in registers: (NWA + NWB) * nr vectors per lane, which
  // fits for up to 10 rows of 3 vectors or 15 rows of 2
  constexpr int kMaxNr = (NWA + NWB <= 10) ? 4 : 2;
  // staged update: as many warps per block (one block per SM) as shared memory holds
  const int staged_stages = 1;
  const int staged_held = (NWB <= NWA) ? NWB : NWA;  // as StagedShape<NWA, NWB, nr>
  const int staged_max_threads = (staged_held * nr <= 15 && NWA * NWB <= 25) ? 512 : 384;
  const size_t per_warp = staged_warp_bytes(NWA + NWB, dim, staged_stages);
  const int staged_warps = (int)std::min<size_t>(staged_max_threads / 32, (227 * 1024) / per_warp);
  // update and scoring both go through the staged pipeline where it fits (scoring measured on
  // the benchmark workload: 1.32 ms staged against 1.72 ms with rows loaded into registers,
  // 2.41 against 3.62 ms for 10+5 columns); the register-resident kernels are the fallback
  const bool want_staged = true;
  const bool staged_fits = vector_ok(dim, A, B) && nr <= 4 && staged_warps >= 2;
  if (!sl.whole() && !staged_fits) {
    printf("word2vecNegSlice needs rows of a multiple of 4 floats, at most 512, 16-byte aligned matrices (dim %d)\n", dim);
    return 1;
  }
  if (want_staged && staged_fits && (neg_staged_enabled() || !sl.whole())) {
    const size_t smem = per_warp * staged_warps;
    // at least 8 columns per warp: a small launch then still applies its updates in several
    // rounds instead of computing every column from the same stale rows
    const int grid = std::max(1, std::min(device_sm_count(), (ncols + 8 * staged_warps - 1) / (8 * staged_warps)));
    cudaError_t e = cudaSuccess;
    switch (nr) {
      case 1: e = launch_neg_staged_any<NWA, NWB, 1>(eval, grid, staged_warps, smem, stream, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot, scratch, retval, fault, sl); break;
      case 2: e = launch_neg_staged_any<NWA, NWB, 2>(eval, grid, staged_warps, smem, stream, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot, scratch, retval, fault, sl); break;
      case 3: e = launch_neg_staged_any<NWA, NWB, 3>(eval, grid, staged_warps, smem, stream, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot, scratch, retval, fault, sl); break;
      default: e = launch_neg_staged_any<NWA, NWB, 4>(eval, grid, staged_warps, smem, stream, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot, scratch, retval, fault, sl); break;
    }
    if (e != cudaSuccess) return (int)e;
    if (!eval) fold_hot_rows(dim, hot, A, B, stream);
  } else if (vector_ok(dim, A, B) && nr <= kMaxNr) {
    const int grid = grid_for(ncols, kNegThreads, eval ? kNegEvalGridBlocks : 8);
    if (eval) {
      switch (nr) {
        case 1: neg_eval_kernel<NWA, NWB, 1><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval, NWA, NWB); break;
        case 2: neg_eval_kernel<NWA, NWB, 2><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval, NWA, NWB); break;
        case 3: neg_eval_kernel<NWA, NWB, (kMaxNr >= 3 ? 3 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval, NWA, NWB); break;
        default: neg_eval_kernel<NWA, NWB, (kMaxNr >= 4 ? 4 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval, NWA, NWB); break;
      }
    } else {
      switch (nr) {
        case 1: neg_update_kernel<NWA, NWB, 1><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot); break;
        case 2: neg_update_kernel<NWA, NWB, 2><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot); break;
        case 3: neg_update_kernel<NWA, NWB, (kMaxNr >= 3 ? 3 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot); break;
        default: neg_update_kernel<NWA, NWB, (kMaxNr >= 4 ? 4 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, hot); break;
      }
      fold_hot_rows(dim, hot, A, B, stream);
    }
  } else {
    const int grid = grid_for(ncols, kGenericThreads, 8);
    if (eval)
      neg_generic_kernel<NWA, NWB, true><<<grid, kGenericThreads, 0, stream>>>(
          dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, scratch, retval);
    else
      neg_generic_kernel<NWA, NWB, false><<<grid, kGenericThreads, 0, stream>>>(
          dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, scratch, retval);
  }
  count_launch(1);
  return (int)cudaGetLastError();
}

static int neg_any(bool eval, int dim, int ncols, const int *ncols_dev, int nwords, int nwa,
                   int nwb, const int *WA, const int *WB, float *A, float *B, float lrate,
                   float vexp, float *retval, const HotRows &hot, EvalScratch *scratch, int *fault,
                   const SliceMap &sl, cudaStream_t stream) {
  if (ncols <= 0) return 0;
  if (dim <= 0) return 1;
  const int which = nwa * 10000 + nwb;
  switch (which) {
    case 50001: return neg_dispatch<5, 1>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, hot, scratch, fault, sl, stream);
    case 50005: return neg_dispatch<5, 5>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, hot, scratch, fault, sl, stream);
    case 100005: return neg_dispatch<10, 5>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, hot, scratch, fault, sl, stream);
    case 50010: return neg_dispatch<5, 10>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, hot, scratch, fault, sl, stream);
    default: return 1;
  }
}

int neg_update_async(int dim, int ncols, const int *ncols_dev, int nwords, int nwa, int nwb,
                     const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, int *fault, const SliceMap &sl, cudaStream_t stream) {
  return neg_any(false, dim, ncols, ncols_dev, nwords, nwa, nwb, WA, WB, A, B, lrate, vexp, nullptr,
                 hot, nullptr, fault, sl, stream);
}

int neg_eval_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                   const int *WB, const float *A, const float *B, float *retval,
                   EvalScratch *scratch, int *fault, const SliceMap &sl, cudaStream_t stream) {
  return neg_any(true, dim, ncols, ncols_dev, 0x7fffffff, nwa, nwb, WA, WB, const_cast<float *>(A),
                 const_cast<float *>(B), 0.f, 0.f, retval, hot_rows_at(nullptr, 0), scratch, fault, sl,
                 stream);
}

bool neg_shape_supported(int nwa, int nwb) {
  const int which = nwa * 10000 + nwb;
  return which == 50001 || which == 50005 || which == 100005 || which == 50010;
}

}  // namespace w2v

// ---------------------------------------------------------------------------
// C entry points with the reference's prototypes (jni/include/MatKernel.hpp:77-85,
// launchers at jni/src/DNN127.cu:1389-1548).  Like the reference they run on
// the calling thread's default stream, wait for completion, and return 0 or a
// cudaError_t; an unsupported shape prints a line and returns 1.
// ---------------------------------------------------------------------------

namespace {

// A scratch set borrowed from the device's pool for the duration of one launcher call.
struct ScratchLease {
  w2v::LaunchScratch *s = nullptr;
  ~ScratchLease() { w2v::release_launch_scratch(s); }
  int acquire() { return w2v::acquire_launch_scratch(&s); }
  // Replica rows with the hot-word share of this launch's own word list, so that the
  // folding period adapts to dense text as it does behind w2v_dobatch.
  int hot_rows(const int *ids, int64_t n, int nwords, w2v::HotRows *out) {
    *out = w2v::hot_rows_at(s->hot_buf, s->hot_buf ? w2v::hot_levels_default() : 0);
    if (out->fold_every <= 0 || n <= 0) return 0;
    out->stats = s->stats;
    return w2v::count_hot_share_async(ids, n, nwords, s->stats, cudaStreamPerThread);
  }
  // Waits for the call's kernels; a staged kernel that gave up waiting for its copies has
  // raised this call's own flag.
  int finish(int launch_err) {
    if (launch_err) return launch_err;
    cudaError_t e = cudaStreamSynchronize(cudaStreamPerThread);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (*reinterpret_cast<volatile int *>(s->fault)) {
      *s->fault = 0;
      return (int)cudaErrorLaunchTimeout;
    }
    return 0;
  }
};

}  // namespace

namespace {

// nslices, islice, nHead, doHead as the reference's slice functions take them; the id's slice
// is id % nslices (BIDMach_CPUMACH.c:85), so islice must lie in [0, nslices)
bool slice_args_ok(const char *name, int islice, int nslices, int nhead) {
  if (nslices >= 1 && islice >= 0 && islice < nslices && nhead >= 0) return true;
  printf("%s bad slice arguments islice %d nslices %d nHead %d\n", name, islice, nslices, nhead);
  return false;
}

int pos_launcher(const char *name, int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A,
                 float *B, float lrate, float vexp, const w2v::SliceMap &sl) {
  if (shift != 5 && shift != 3 && shift != 2) {
    printf("%s unsupport size %d\n", name, shift);
    return 1;
  }
  if (nrows > 1280) {
    printf("%s too many rows %d\n", name, nrows);
    return 1;
  }
  if (ncols <= 0) return 0;
  ScratchLease lease;
  int err = lease.acquire();
  if (err) return err;
  w2v::HotRows hot;
  err = lease.hot_rows(W, ncols, 0x7fffffff, &hot);
  if (err) return err;
  return lease.finish(w2v::pos_update_async(nrows, ncols, nullptr, shift, W, LB, UB, A, B, lrate,
                                            vexp, hot, sl, cudaStreamPerThread));
}

int neg_launcher(int nrows, int ncols, int nwords, int nwa, int nwb, int *WA, int *WB, float *A,
                 float *B, float lrate, float vexp, const w2v::SliceMap &sl) {
  if (!w2v::neg_shape_supported(nwa, nwb)) {
    printf("word2vec unsupport size combination %d %d\n", nwa, nwb);
    return 1;
  }
  if (ncols <= 0) return 0;
  ScratchLease lease;
  int err = lease.acquire();
  if (err) return err;
  w2v::HotRows hot;
  err = lease.hot_rows(WB, (int64_t)ncols * nwb, nwords, &hot);
  if (err) return err;
  return lease.finish(w2v::neg_update_async(nrows, ncols, nullptr, nwords, nwa, nwb, WA, WB, A, B,
                                            lrate, vexp, hot, lease.s->fault, sl, cudaStreamPerThread));
}

int eval_pos_launcher(const char *name, int nrows, int ncols, int shift, int *W, int *LB, int *UB,
                      float *A, float *B, float *Retval, const w2v::SliceMap &sl) {
  if (shift != 5 && shift != 3 && shift != 2) {
    printf("%s unsupport size %d\n", name, shift);
    return 1;
  }
  if (nrows > 1280) {
    printf("%s nrows too large %d\n", name, nrows);
    return 1;
  }
  if (ncols <= 0) return 0;
  ScratchLease lease;
  int err = lease.acquire();
  if (err) return err;
  return lease.finish(w2v::pos_eval_async(nrows, ncols, nullptr, shift, W, LB, UB, A, B, Retval,
                                          lease.s->eval, sl, cudaStreamPerThread));
}

int eval_neg_launcher(const char *name, int nrows, int ncols, int nwa, int nwb, int *WA, int *WB,
                      float *A, float *B, float *Retval, const w2v::SliceMap &sl) {
  if (!w2v::neg_shape_supported(nwa, nwb)) {
    printf("%s unsupport size combination %d %d\n", name, nwa, nwb);
    return 1;
  }
  if (ncols <= 0) return 0;
  ScratchLease lease;
  int err = lease.acquire();
  if (err) return err;
  return lease.finish(w2v::neg_eval_async(nrows, ncols, nullptr, nwa, nwb, WA, WB, A, B, Retval,
                                          lease.s->eval, lease.s->fault, sl, cudaStreamPerThread));
}

}  // namespace

extern "C" {

int word2vecPos(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                float lrate, float vexp) {
  return pos_launcher("word2vecPos", nrows, ncols, shift, W, LB, UB, A, B, lrate, vexp,
                      w2v::whole_vocabulary());
}

int word2vecNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                float lrate, float vexp) {
  return neg_launcher(nrows, ncols, 0x7fffffff, nwa, nwb, WA, WB, A, B, lrate, vexp,
                      w2v::whole_vocabulary());
}

int word2vecNegFilt(int nrows, int ncols, int nwords, int nwa, int nwb, int *WA, int *WB, float *A,
                    float *B, float lrate, float vexp) {
  return neg_launcher(nrows, ncols, nwords, nwa, nwb, WA, WB, A, B, lrate, vexp, w2v::whole_vocabulary());
}

int word2vecEvalPos(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                    float *Retval) {
  return eval_pos_launcher("word2vecEvalPos", nrows, ncols, shift, W, LB, UB, A, B, Retval,
                           w2v::whole_vocabulary());
}

int word2vecEvalNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                    float *Retval) {
  return eval_neg_launcher("word2vecEvalNeg", nrows, ncols, nwa, nwb, WA, WB, A, B, Retval,
                           w2v::whole_vocabulary());
}

// Vocabulary slices (the device forms of CPUMACH.word2vecPosSlice / word2vecNegSlice and of
// Word2Vec.evalPosCPUslice / evalNegCPUslice).
int word2vecPosSlice(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                     float lrate, float vexp, int islice, int nslices, int nHead, int doHead) {
  if (!slice_args_ok("word2vecPosSlice", islice, nslices, nHead)) return 1;
  return pos_launcher("word2vecPosSlice", nrows, ncols, shift, W, LB, UB, A, B, lrate, vexp,
                      w2v::SliceMap{nHead, nslices, islice, doHead});
}

int word2vecNegSlice(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                     float lrate, float vexp, int islice, int nslices, int nHead, int doHead) {
  if (!slice_args_ok("word2vecNegSlice", islice, nslices, nHead)) return 1;
  return neg_launcher(nrows, ncols, 0x7fffffff, nwa, nwb, WA, WB, A, B, lrate, vexp,
                      w2v::SliceMap{nHead, nslices, islice, doHead});
}

int word2vecEvalPosSlice(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                         float *Retval, int islice, int nslices, int nHead) {
  if (!slice_args_ok("word2vecEvalPosSlice", islice, nslices, nHead)) return 1;
  return eval_pos_launcher("word2vecEvalPosSlice", nrows, ncols, shift, W, LB, UB, A, B, Retval,
                           w2v::SliceMap{nHead, nslices, islice, 1});
}

int word2vecEvalNegSlice(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                         float *Retval, int islice, int nslices, int nHead) {
  if (!slice_args_ok("word2vecEvalNegSlice", islice, nslices, nHead)) return 1;
  return eval_neg_launcher("word2vecEvalNegSlice", nrows, ncols, nwa, nwb, WA, WB, A, B, Retval,
                           w2v::SliceMap{nHead, nslices, islice, 1});
}

long long w2v_launch_count(void) { return w2v::launch_count(); }

}  // extern "C"
