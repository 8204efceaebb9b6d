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
// Work decomposition: one warp per centre (Pos) or per column (Neg); the rows
// of the unit live in registers as 128-bit vectors; dot products are reduced
// with warp shuffles; grids are sized to fill every SM and stride over the
// minibatch.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "w2v_device.cuh"
#include "w2v_internal.h"

namespace w2v {

constexpr int kPosThreads = 256;
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

template <int NR>
__global__ void __launch_bounds__(kPosThreads)
    pos_update_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                      const int *__restrict__ W, const int *__restrict__ LB,
                      const int *__restrict__ UB, float *A, float *B, float lrate, float vexp) {
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;

  for (int i = gwarp; i < ncols; i += nwarps) {
    const int wc = W[i];
    if (wc < 0) continue;
    const int lb = max(LB[i], -skip), ub = min(UB[i], skip);
    const int wx = window_word(W, i, lb, ub, ncols, lane);
    unsigned todo = __ballot_sync(kFullMask, wx >= 0);
    if (todo == 0) continue;
    // lane 31 never carries a context (the window has at most 31 offsets), so
    // it evaluates the centre's scale while the others do their context's.
    const int sid = (lane == 31) ? wc : wx;
    const float sc = (sid >= 0) ? freq_scale(sid, vexp) : 0.f;
    const float sa = __shfl_sync(kFullMask, sc, 31);

    Row<NR> a, da;
    row_load(a, A, wc, dim, nvec, lane);
    row_zero(da);
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const int w = __shfl_sync(kFullMask, wx, src);
      const float sb = __shfl_sync(kFullMask, sc, src);
      Row<NR> b;
      row_load(b, B, w, dim, nvec, lane);
      const float g = lrate * (1.0f - sigmoid_guard(warp_sum(row_dot_partial(a, b))));
      row_axpy(da, sa * g, b);
      Row<NR> db;
      row_zero(db);
      row_axpy(db, sb * g, a);
      row_red(B, w, dim, nvec, lane, db);
    }
    row_red(A, wc, dim, nvec, lane, da);
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

template <int NR>
__global__ void __launch_bounds__(kPosThreads)
    pos_eval_kernel(int dim, int ncols, const int *__restrict__ ncols_dev, int skip,
                    const int *__restrict__ W, const int *__restrict__ LB,
                    const int *__restrict__ UB, const float *__restrict__ A,
                    const float *__restrict__ B, EvalScratch *scratch, float *retval) {
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
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
    if (todo == 0) continue;
    Row<NR> a;
    row_load(a, A, wc, dim, nvec, lane);
    float mine = 0.f;
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const int w = __shfl_sync(kFullMask, wx, src);
      Row<NR> b;
      row_load(b, B, w, dim, nvec, lane);
      const float p = warp_sum(row_dot_partial(a, b));
      if (lane == src) mine = p;
    }
    // each context lane scores its own pair (networks/Word2Vec.scala:995)
    if (wx >= 0) acc += log(fmax((double)sigmoid_guard(mine), 1e-20));
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
    if (wx >= 0) acc += log(fmax((double)sigmoid_guard(mine), 1e-20));
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
                      float lrate, float vexp) {
  using S = Spread<NWA * NWB>;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;

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
#pragma unroll
    for (int idx = NWA * NWB - 1; idx >= 0; idx--)
      g[idx] = __shfl_sync(kFullMask, p[S::slot_of(idx)], S::lane_of(idx));

#pragma unroll
    for (int j = 0; j < NWA; j++) {
      const float sa = __shfl_sync(kFullMask, mysc, j);
      Row<NR> d;
      row_zero(d);
#pragma unroll
      for (int k = 0; k < NWB; k++) row_axpy(d, sa * g[j * NWB + k], b[k]);
      if (wa[j] >= 0) row_red(A, wa[j], dim, nvec, lane, d);
    }
#pragma unroll
    for (int k = 0; k < NWB; k++) {
      const float sb = __shfl_sync(kFullMask, mysc, NWA + k);
      Row<NR> d;
      row_zero(d);
#pragma unroll
      for (int j = 0; j < NWA; j++) row_axpy(d, sb * g[j * NWB + k], a[j]);
      if (wb[k] >= 0) row_red(B, wb[k], dim, nvec, lane, d);
    }
  }
}

template <int NWA, int NWB, int NR>
__global__ void __launch_bounds__(kNegThreads)
    neg_eval_kernel(int dim, int ncols, const int *__restrict__ ncols_dev,
                    const int *__restrict__ WA, const int *__restrict__ WB,
                    const float *__restrict__ A, const float *__restrict__ B,
                    EvalScratch *scratch, float *retval) {
  using S = Spread<NWA * NWB>;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (ncols_dev) ncols = *ncols_dev;
  double acc = 0.0;

  for (int col = gwarp; col < ncols; col += nwarps) {
    const int myw = column_word<NWA, NWB>(WA, WB, col, 0x7fffffff, lane);
    Row<NR> a[NWA], b[NWB];
#pragma unroll
    for (int j = 0; j < NWA; j++)
      row_load(a[j], A, __shfl_sync(kFullMask, myw, j), dim, nvec, lane);
#pragma unroll
    for (int k = 0; k < NWB; k++)
      row_load(b[k], B, __shfl_sync(kFullMask, myw, NWA + k), dim, nvec, lane);
    float p[NWA * NWB];
    column_dots<NWA, NWB, NR>(a, b, p, lane);
#pragma unroll
    for (int q = 0; q < S::FIN; q++) {
      const unsigned valid = spread_valid_mask<NWA * NWB>(q);
      if ((valid >> lane) & 1u)
        acc += log(fmax((double)(1.0f - sigmoid_guard(p[q])), 1e-20));
    }
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

    if (EVAL) {
#pragma unroll
      for (int q = 0; q < S::FIN; q++) {
        const unsigned valid = spread_valid_mask<NWA * NWB>(q);
        if ((valid >> lane) & 1u)
          acc += log(fmax((double)(1.0f - sigmoid_guard(p[q])), 1e-20));
      }
      continue;
    }

#pragma unroll
    for (int q = 0; q < S::FIN; q++) p[q] = -lrate * sigmoid_guard(p[q]);
    float g[NWA * NWB];
#pragma unroll
    for (int idx = NWA * NWB - 1; idx >= 0; idx--)
      g[idx] = __shfl_sync(kFullMask, p[S::slot_of(idx)], S::lane_of(idx));
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
  if (EVAL) finish_eval_sum(acc, scratch, retval);
}

// ---------------------------------------------------------------------------
// Host side: device facts, scratch, dispatch
// ---------------------------------------------------------------------------

static std::atomic<long long> g_launches{0};

long long launch_count() { return g_launches.load(); }
void count_launch(int n) { g_launches.fetch_add(n); }

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
  return cached_sms;
}

// One small zero-initialised accumulator per (host thread, device): the eval
// kernels sum in double there and re-arm it themselves, so concurrent callers
// on different threads or devices never share it.
int eval_scratch(EvalScratch **out) {
  constexpr int kMaxDev = 64;
  thread_local EvalScratch *per_dev[kMaxDev] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDev) return (int)cudaErrorInvalidDevice;
  if (!per_dev[dev]) {
    EvalScratch *p = nullptr;
    e = cudaMalloc(&p, 256);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(p, 0, 256);
    if (e != cudaSuccess) return (int)e;
    per_dev[dev] = p;
  }
  *out = per_dev[dev];
  return 0;
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

int pos_update_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W,
                     const int *LB, const int *UB, float *A, float *B, float lrate, float vexp,
                     cudaStream_t stream) {
  if (ncols <= 0) return 0;
  if (skip < 1 || skip > 15) return 1;
  if (vector_ok(dim, A, B)) {
    const int nr = (dim / 4 + 31) / 32;
    const int grid = grid_for(ncols, kPosThreads, 8);
    W2V_NR_SWITCH(nr, (pos_update_kernel<NR><<<grid, kPosThreads, 0, stream>>>(
                          dim, ncols, ncols_dev, skip, W, LB, UB, A, B, lrate, vexp)));
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
                   cudaStream_t stream) {
  if (ncols <= 0) return 0;
  if (skip < 1 || skip > 15) return 1;
  EvalScratch *scratch = nullptr;
  int err = eval_scratch(&scratch);
  if (err) return err;
  if (vector_ok(dim, A, B)) {
    const int nr = (dim / 4 + 31) / 32;
    const int grid = grid_for(ncols, kPosThreads, 8);
    W2V_NR_SWITCH(nr, (pos_eval_kernel<NR><<<grid, kPosThreads, 0, stream>>>(
                          dim, ncols, ncols_dev, skip, W, LB, UB, A, B, scratch, retval)));
  } else {
    const int grid = grid_for(ncols, kGenericThreads, 16);
    pos_eval_generic_kernel<<<grid, kGenericThreads, 0, stream>>>(
        dim, ncols, ncols_dev, skip, W, LB, UB, A, B, scratch, retval);
  }
  count_launch(1);
  return (int)cudaGetLastError();
}

template <int NWA, int NWB>
static int neg_dispatch(bool eval, int dim, int ncols, const int *ncols_dev, int nwords,
                        const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                        float *retval, cudaStream_t stream) {
  EvalScratch *scratch = nullptr;
  if (eval) {
    int err = eval_scratch(&scratch);
    if (err) return err;
  }
  const int nr = (dim / 4 + 31) / 32;
  // rows of a column live in registers: (NWA + NWB) * nr vectors per lane, which
  // fits for up to 10 rows of 3 vectors or 15 rows of 2
  constexpr int kMaxNr = (NWA + NWB <= 10) ? 4 : 2;
  if (vector_ok(dim, A, B) && nr <= kMaxNr) {
    const int grid = grid_for(ncols, kNegThreads, 8);
    if (eval) {
      switch (nr) {
        case 1: neg_eval_kernel<NWA, NWB, 1><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval); break;
        case 2: neg_eval_kernel<NWA, NWB, 2><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval); break;
        case 3: neg_eval_kernel<NWA, NWB, (kMaxNr >= 3 ? 3 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval); break;
        default: neg_eval_kernel<NWA, NWB, (kMaxNr >= 4 ? 4 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, WA, WB, A, B, scratch, retval); break;
      }
    } else {
      switch (nr) {
        case 1: neg_update_kernel<NWA, NWB, 1><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp); break;
        case 2: neg_update_kernel<NWA, NWB, 2><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp); break;
        case 3: neg_update_kernel<NWA, NWB, (kMaxNr >= 3 ? 3 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp); break;
        default: neg_update_kernel<NWA, NWB, (kMaxNr >= 4 ? 4 : 1)><<<grid, kNegThreads, 0, stream>>>(dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp); break;
      }
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
                   float vexp, float *retval, cudaStream_t stream) {
  if (ncols <= 0) return 0;
  if (dim <= 0) return 1;
  const int which = nwa * 10000 + nwb;
  switch (which) {
    case 50001: return neg_dispatch<5, 1>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, stream);
    case 50005: return neg_dispatch<5, 5>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, stream);
    case 100005: return neg_dispatch<10, 5>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, stream);
    case 50010: return neg_dispatch<5, 10>(eval, dim, ncols, ncols_dev, nwords, WA, WB, A, B, lrate, vexp, retval, stream);
    default: return 1;
  }
}

int neg_update_async(int dim, int ncols, const int *ncols_dev, int nwords, int nwa, int nwb,
                     const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                     cudaStream_t stream) {
  return neg_any(false, dim, ncols, ncols_dev, nwords, nwa, nwb, WA, WB, A, B, lrate, vexp, nullptr,
                 stream);
}

int neg_eval_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                   const int *WB, const float *A, const float *B, float *retval,
                   cudaStream_t stream) {
  return neg_any(true, dim, ncols, ncols_dev, 0x7fffffff, nwa, nwb, WA, WB, const_cast<float *>(A),
                 const_cast<float *>(B), 0.f, 0.f, retval, stream);
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

static int finish_sync(int launch_err) {
  if (launch_err) return launch_err;
  cudaError_t e = cudaStreamSynchronize(cudaStreamPerThread);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

extern "C" {

int word2vecPos(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                float lrate, float vexp) {
  if (shift != 5 && shift != 3 && shift != 2) {
    printf("word2vecPos unsupport size %d\n", shift);
    return 1;
  }
  if (nrows > 1280) {
    printf("word2vecPos too many rows %d\n", nrows);
    return 1;
  }
  return finish_sync(w2v::pos_update_async(nrows, ncols, nullptr, shift, W, LB, UB, A, B, lrate,
                                           vexp, cudaStreamPerThread));
}

int word2vecNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                float lrate, float vexp) {
  if (!w2v::neg_shape_supported(nwa, nwb)) {
    printf("word2vec unsupport size combination %d %d\n", nwa, nwb);
    return 1;
  }
  return finish_sync(w2v::neg_update_async(nrows, ncols, nullptr, 0x7fffffff, nwa, nwb, WA, WB, A,
                                           B, lrate, vexp, cudaStreamPerThread));
}

int word2vecNegFilt(int nrows, int ncols, int nwords, int nwa, int nwb, int *WA, int *WB, float *A,
                    float *B, float lrate, float vexp) {
  if (!w2v::neg_shape_supported(nwa, nwb)) {
    printf("word2vec unsupport size combination %d %d\n", nwa, nwb);
    return 1;
  }
  return finish_sync(w2v::neg_update_async(nrows, ncols, nullptr, nwords, nwa, nwb, WA, WB, A, B,
                                           lrate, vexp, cudaStreamPerThread));
}

int word2vecEvalPos(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                    float *Retval) {
  if (shift != 5 && shift != 3 && shift != 2) {
    printf("word2vecEvalPos unsupport size %d\n", shift);
    return 1;
  }
  if (nrows > 1280) {
    printf("word2vecEvalPos nrows too large %d\n", nrows);
    return 1;
  }
  return finish_sync(w2v::pos_eval_async(nrows, ncols, nullptr, shift, W, LB, UB, A, B, Retval,
                                         cudaStreamPerThread));
}

int word2vecEvalNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                    float *Retval) {
  if (!w2v::neg_shape_supported(nwa, nwb)) {
    printf("word2vecEvalNeg unsupport size combination %d %d\n", nwa, nwb);
    return 1;
  }
  return finish_sync(w2v::neg_eval_async(nrows, ncols, nullptr, nwa, nwb, WA, WB, A, B, Retval,
                                         cudaStreamPerThread));
}

long long w2v_launch_count(void) { return w2v::launch_count(); }

}  // extern "C"
