// Whole-minibatch path: the device version of Word2Vec.wordMats / dobatch /
// evalbatch (networks/Word2Vec.scala:167-278) on top of the four kernels.
//
// Pipeline for one minibatch of `ncols` tokens (all on one stream):
//   1. words_bounds_kernel   subsampling mask + window bounds      (:216-237)
//   2. count_pairs_kernel    good contexts per centre              (:283-302)
//   3. exclusive scan        start of each centre's contexts
//   4. fill_pairs_kernel     ordered context list + permutation keys (:309-330, :254-255)
//   5. radix sort            permutation = stable descending key order (:256-259)
//   6. negative_ids_kernel   min(V-1, int(V * u^expt))             (:264-265, :356)
//   7. Pos / Neg update kernels, or the two eval kernels
//
// Every step is a deterministic map of the token matrix and of four arrays of
// uniform draws, so with caller-supplied draws the outputs can be compared bit
// for bit with the CPU path.  Without them the draws come from Philox4x32-10
// (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed
// by (seed, batch id), generated inside the kernels that consume them.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include <nvtx3/nvToolsExt.h>

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "../../include/bidmach_b200.h"
#include "w2v_internal.h"

namespace w2v {

// ---------------------------------------------------------------------------
// Philox4x32-10
// ---------------------------------------------------------------------------
struct PhiloxOut {
  uint32_t v[4];
};

__host__ __device__ inline PhiloxOut philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2,
                                                   uint32_t c3, uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int r = 0; r < 10; r++) {
    uint64_t p0 = (uint64_t)M0 * c0, p1 = (uint64_t)M1 * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  PhiloxOut o;
  o.v[0] = c0; o.v[1] = c1; o.v[2] = c2; o.v[3] = c3;
  return o;
}

// 24 random bits -> fp32 in [0, 1)
__host__ __device__ inline float u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }

enum : uint32_t { kStreamSampleWindow = 1, kStreamPermute = 2, kStreamNegs = 3, kStreamInit = 4 };

struct Rng {
  uint32_t k0, k1, batch;
};

// ---------------------------------------------------------------------------
// Keyed permutation of [0, n) without a sort.  f(x) = four rounds of
// x = (x * a + c) mod 2^b;  x ^= x >> ceil(b / 2)  is a bijection of [0, 2^b)
// (an odd multiplier and a right xor-shift are both invertible), b being the
// bit length of n - 1; following f from i until the value drops below n
// ("cycle walking") restricts it to a bijection of [0, n).  2^b < 2n, so a walk
// takes under two steps on average.  The eight constants come from one Philox
// block pair per minibatch.
// ---------------------------------------------------------------------------
struct PermKeys {
  uint32_t a[4], c[4];
};

__host__ __device__ inline uint32_t permute_index(uint32_t i, uint32_t n, const PermKeys &k) {
  if (n < 2) return 0;
  int b = 0;
  while (b < 32 && ((n - 1) >> b) != 0) b++;
  const uint32_t mask = (b >= 32) ? 0xFFFFFFFFu : ((1u << b) - 1u);
  const int sh = (b + 1) >> 1;
  uint32_t x = i;
  do {
#pragma unroll
    for (int r = 0; r < 4; r++) {
      x = (x * k.a[r] + k.c[r]) & mask;
      x ^= x >> sh;
    }
  } while (x >= n);
  return x;
}

// The inverse of permute_index: the place i with permute_index(i, n, k) == p.  Every round is
// undone in reverse order (x ^= x >> sh is its own inverse because sh >= b / 2; the affine step
// with the multiplier's inverse modulo 2^32, which is also its inverse modulo 2^b), and walking
// the inverse map from p until the value drops below n undoes the cycle walk.
struct PermInverse {
  uint32_t ainv[4], c[4];
};

__host__ __device__ inline uint32_t unpermute_index(uint32_t p, uint32_t n, const PermInverse &k) {
  if (n < 2) return 0;
  int b = 0;
  while (b < 32 && ((n - 1) >> b) != 0) b++;
  const uint32_t mask = (b >= 32) ? 0xFFFFFFFFu : ((1u << b) - 1u);
  const int sh = (b + 1) >> 1;
  uint32_t x = p;
  do {
#pragma unroll
    for (int r = 3; r >= 0; r--) {
      x ^= x >> sh;
      x = ((x - k.c[r]) * k.ainv[r]) & mask;
    }
  } while (x >= n);
  return x;
}

// ---------------------------------------------------------------------------
// Preprocessing kernels
// ---------------------------------------------------------------------------

// words[i] = id if (id < vocab and u1 < sqrt(x) + x, x = float(id+1) * salpha) else -1;
// ub = min(nskip, int(u2 * nskip) + 1) clipped to the sentence; lb likewise.
// Sentence clipping only ever matters within nskip positions, so each thread
// looks at most nskip tokens back and forth instead of running a segmented scan.
__global__ void words_bounds_kernel(int ncols, const int *__restrict__ tokens, int wrow, int vocab,
                                    int nskip, float salpha, const float *__restrict__ usample,
                                    const float *__restrict__ uwindow, Rng rng,
                                    int *__restrict__ words, int *__restrict__ lb,
                                    int *__restrict__ ub, int *__restrict__ stats) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool good = false;
  int id = -1;
  if (i < ncols) {
    const int srow = 1 - wrow;
    id = tokens[2 * i + wrow];
    const int sid = tokens[2 * i + srow];
    float u1, u2;
    if (usample == nullptr || uwindow == nullptr) {
      PhiloxOut r = philox4x32_10((uint32_t)i, 0u, kStreamSampleWindow, rng.batch, rng.k0, rng.k1);
      u1 = u01(r.v[0]);
      u2 = u01(r.v[1]);
    }
    if (usample) u1 = usample[i];
    if (uwindow) u2 = uwindow[i];

    const float x = __fmul_rn((float)(id + 1), salpha);
    const float thr = __fadd_rn(__fsqrt_rn(x), x);
    good = (id < vocab) && (u1 < thr);
    words[i] = good ? id : -1;

    int ubr = (int)__fmul_rn(u2, (float)nskip) + 1;
    ubr = min(ubr, nskip);
    int back = 0;
    while (back < nskip && i - back - 1 >= 0 && tokens[2 * (i - back - 1) + srow] == sid) back++;
    int fwd = 0;
    while (fwd < nskip && i + fwd + 1 < ncols && tokens[2 * (i + fwd + 1) + srow] == sid) fwd++;
    lb[i] = max(-ubr, -back);
    ub[i] = min(ubr, fwd);
  }
  // kept tokens, and kept tokens of the most frequent word (id 0): the update kernels
  // derive their folding period from this share; one pair of atomics per block
  const int k = __syncthreads_count(good), z = __syncthreads_count(good && id == 0);
  if (threadIdx.x == 0) {
    if (k) atomicAdd(&stats[0], k);
    if (z) atomicAdd(&stats[1], z);
  }
}

__global__ void count_pairs_kernel(int ncols, const int *__restrict__ words,
                                   const int *__restrict__ lb, const int *__restrict__ ub,
                                   int *__restrict__ cnt) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ncols) return;
  int n = 0;
  if (words[i] >= 0) {
    const int hi = ub[i];
    for (int j = lb[i]; j <= hi; j++)
      if (j != 0 && words[i + j] >= 0) n++;
  }
  cnt[i] = n;
}

// counts[0] = number of pairs, counts[1] = pairs / nreuse
__global__ void totals_kernel(int ncols, const int *__restrict__ cnt, const int *__restrict__ off,
                              int nreuse, int *__restrict__ counts) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int total = (ncols > 0) ? off[ncols - 1] + cnt[ncols - 1] : 0;
    counts[0] = total;
    counts[1] = total / nreuse;
  }
}

// Context words in (centre ascending, offset ascending) order, each with its
// permutation key.  The reference turns a uniform u into the key (u + 1) - 1
// in fp32 (Word2Vec.scala:255), i.e. u rounded to a multiple of 2^-23; the key
// is stored as that multiple, an integer in [0, 2^23], which sorts identically.
__global__ void fill_pairs_kernel(int ncols, int nskip, const int *__restrict__ words,
                                  const int *__restrict__ lb, const int *__restrict__ ub,
                                  const int *__restrict__ off, const float *__restrict__ upermute,
                                  Rng rng, int *__restrict__ ctx, uint32_t *__restrict__ keys) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ncols) return;
  if (words[i] < 0) return;
  int at = off[i];
  const int hi = ub[i];
  PhiloxOut r;
  int have = -1;
  for (int j = lb[i]; j <= hi; j++) {
    if (j == 0) continue;
    const int w = words[i + j];
    if (w < 0) continue;
    const int row = (j < 0) ? j + nskip : j + nskip - 1;
    ctx[at] = w;
    if (keys) {
      float u;
      if (upermute) {
        u = upermute[(int64_t)i * (2 * nskip) + row];
      } else {
        if ((row >> 2) != have) {
          have = row >> 2;
          r = philox4x32_10((uint32_t)i, (uint32_t)have, kStreamPermute, rng.batch, rng.k0, rng.k1);
        }
        u = u01(r.v[row & 3]);
      }
      const float key = __fadd_rn(__fadd_rn(u, 1.0f), -1.0f);
      keys[at] = (uint32_t)__fmul_rn(key, 8388608.0f);
    }
    at++;
  }
}

// out[i] = ctx[perm(i)] for the first groups * nreuse places of the keyed
// permutation of the counts[0] pairs (counts as totals_kernel leaves them).
__global__ void shuffle_contexts_kernel(const int *__restrict__ counts, int nreuse, PermKeys keys,
                                        const int *__restrict__ ctx, int *__restrict__ out) {
  const uint32_t n = (uint32_t)counts[0];
  const uint32_t m = (uint32_t)counts[1] * (uint32_t)nreuse;
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < m; i += stride)
    out[i] = ctx[permute_index(i, n, keys)];
}

// The shuffled context matrix straight from the token windows, without the ordered pair list in
// between: pair p of the (centre ascending, offset ascending) order belongs at place
// unpermute_index(p) of WB, so the thread of a centre sends each of its contexts there (places at
// or beyond groups * nreuse are the dropped tail).  Same WB, bit for bit, as fill_pairs_kernel
// followed by shuffle_contexts_kernel, with coalesced reads and no 24 MB list written and
// gathered again.
__global__ void scatter_pairs_kernel(int ncols, const int *__restrict__ counts, int nreuse,
                                     PermInverse inv, const int *__restrict__ words,
                                     const int *__restrict__ lb, const int *__restrict__ ub,
                                     const int *__restrict__ off, int *__restrict__ wb) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ncols) return;
  if (words[i] < 0) return;
  const uint32_t n = (uint32_t)counts[0];
  const uint32_t m = (uint32_t)counts[1] * (uint32_t)nreuse;
  uint32_t p = (uint32_t)off[i];
  const int hi = ub[i];
  for (int j = lb[i]; j <= hi; j++) {
    if (j == 0) continue;
    const int w = words[i + j];
    if (w < 0) continue;
    const uint32_t place = unpermute_index(p++, n, inv);
    if (place < m) wb[place] = w;
  }
}

// n draws, or counts[1] * nneg of them when the count is only known on the device
__global__ void negative_ids_kernel(int64_t n, const int *__restrict__ counts, int nneg,
                                    const float *__restrict__ unegs, Rng rng, int vocab,
                                    float expt, int *__restrict__ out) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (counts) n = (int64_t)counts[1] * nneg;
  if (q >= n) return;
  float u;
  if (unegs) {
    u = unegs[q];
  } else {
    const uint64_t blk = (uint64_t)q >> 2;
    PhiloxOut r = philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), kStreamNegs, rng.batch,
                                rng.k0, rng.k1);
    u = u01(r.v[q & 3]);
  }
  const double v = (double)vocab * pow((double)u, (double)expt);
  const int id = (v >= 2147483647.0) ? 2147483647 : (int)v;
  out[q] = min(id, vocab - 1);
}

__global__ void init_model_kernel(int64_t n, int dim, Rng rng, float *__restrict__ B) {
  const int64_t blk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t e = blk * 4;
  if (e >= n) return;
  PhiloxOut r = philox4x32_10((uint32_t)blk, (uint32_t)((uint64_t)blk >> 32), kStreamInit, 0u,
                              rng.k0, rng.k1);
  const float fd = (float)dim;
#pragma unroll
  for (int k = 0; k < 4; k++)
    if (e + k < n) B[e + k] = __fdiv_rn(__fadd_rn(u01(r.v[k]), -0.5f), fd);
}

// theta += avg - base, 16 bytes per thread and trip (all three 16-byte aligned)
__global__ void apply_average_kernel(float4 *__restrict__ theta, const float4 *__restrict__ base,
                                     const float4 *__restrict__ avg, int64_t nvec) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 t = theta[i];
    const float4 b = base[i], a = avg[i];
    t.x += a.x - b.x;
    t.y += a.y - b.y;
    t.z += a.z - b.z;
    t.w += a.w - b.w;
    theta[i] = t;
  }
}

}  // namespace w2v

// ---------------------------------------------------------------------------
// Context
// ---------------------------------------------------------------------------
struct w2v_ctx {
  w2v_opts o;
  int ncols;
  int device;
  int64_t max_pairs;
  float expt, salpha;
  int64_t first_pos;
  // device
  int *tokens, *words, *lb, *ub, *cnt, *off, *counts;
  // host-minibatch entry points: two token buffers filled on a copy stream, so that
  // the upload of the next minibatch runs beside the kernels of the current one
  int *tokens_in[2];
  cudaStream_t copy_stream;
  cudaEvent_t ev_copied[2], ev_read[2];   // upload done / the preprocessing has read the buffer
  int read_recorded[2];
  uint64_t host_calls;
  int *ctx_in, *ctx_out, *wa;
  uint32_t *key_in, *key_out;
  float *retvals;  // [0] positive, [1] negative
  float *hot_buf;  // replica rows of the hot ids
  w2v::HotRows hot;
  w2v::EvalScratch *eval;  // accumulator of the scoring kernels (inside `counts`)
  int *fault_host;         // pinned: set by a staged kernel that gave up waiting for its copies
  int sm_reserve;          // SMs the update kernels leave free (w2v_reserve_sms)
  w2v::SliceMap slice;     // which rows of the vocabulary the caller's matrices hold (w2v_set_slice)
  cudaEvent_t ev_pos;      // end of the latest positive update (w2v_wait_pos)
  int pos_recorded;
  int have_list;           // the latest preprocessing wrote the ordered pair list (ctx_in)
  cudaEvent_t neg_wait;    // the next negative update waits for this event first (w2v_wait_before_neg)
  void *cub_tmp;
  size_t cub_tmp_bytes;
  // pinned host
  int *counts_host;     // [kRing][2]: pairs, groups of the batch that used the slot
  float *retvals_host;
  // results of the latest wordmats: on the device in counts[0..1], on the host
  // once settle_counts has waited for their copy
  int64_t npairs;
  int ngroups;
  int counts_pending;
  cudaEvent_t ev_counts;
  // Batches rotate through kRing slots, so that the host can run ahead of the
  // device by several minibatches.  Phase timers (off by default): events at
  // the phase boundaries of a slot's batch, harvested before the slot is used
  // again or when the timers are read.
  uint64_t nbatch;
  int slot;
  int timing_on;
  cudaEvent_t ev[4][5];
  int ev_state[4];      // 0 none, 1 train batch, 2 eval batch
  cudaStream_t ev_stream;
  w2v_timing acc;
};
constexpr int kRing = 4;

#define W2V_CHECK(call)                    \
  do {                                     \
    cudaError_t e_ = (call);               \
    if (e_ != cudaSuccess) return (int)e_; \
  } while (0)

static w2v::Rng make_rng(const w2v_opts &o, uint64_t batch_id) {
  w2v::Rng r;
  r.k0 = (uint32_t)o.seed;
  r.k1 = (uint32_t)(o.seed >> 32);
  r.batch = (uint32_t)batch_id;
  return r;
}

static void mark(w2v_ctx *c, int k, cudaStream_t stream) {
  if (c->timing_on) cudaEventRecord(c->ev[c->slot][k], stream);
}

// Named range on the host thread for timeline tools (NVTX; costs nothing when no tool is attached).
// The ranges follow the reference's addTime phases (networks/Word2Vec.scala:168-268): "w2v.wordmats"
// covers its phases 1-7 (subsampling and bounds 1-4, pair list 5, permutation 6, negatives 7),
// "w2v.pos" / "w2v.neg" its phases 8 / 9 and "w2v.evalpos" / "w2v.evalneg" its phases 10 / 11.
struct Range {
  explicit Range(const char *name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
};

// Waits for the pair and group counts of the latest wordmats to reach the host.
static int settle_counts(w2v_ctx *c) {
  if (!c->counts_pending) return 0;
  cudaError_t e = cudaEventSynchronize(c->ev_counts);
  if (e != cudaSuccess) return (int)e;
  c->npairs = c->counts_host[2 * c->slot];
  c->ngroups = c->counts_host[2 * c->slot + 1];
  c->counts_pending = 0;
  return 0;
}

// Adds the phase durations and counts of the batch that used `slot`; waits for
// that batch to finish if it has not yet.
static void harvest(w2v_ctx *c, int slot) {
  const int kind = c->ev_state[slot];
  if (!kind) return;
  c->ev_state[slot] = 0;
  if (cudaEventSynchronize(c->ev[slot][4]) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  float ms[4] = {0, 0, 0, 0};
  bool ok = true;
  for (int k = 0; k < 4; k++)
    ok = ok && cudaEventElapsedTime(&ms[k], c->ev[slot][k], c->ev[slot][k + 1]) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    return;
  }
  const int64_t pairs = c->counts_host[2 * slot], groups = c->counts_host[2 * slot + 1];
  c->acc.prep_ms += ms[0];
  c->acc.permute_ms += ms[1];
  if (kind == 1) {
    c->acc.pos_ms += ms[2];
    c->acc.neg_ms += ms[3];
    c->acc.train_batches += 1;
    c->acc.pairs += pairs;
    c->acc.groups += groups;
  } else {
    c->acc.evalpos_ms += ms[2];
    c->acc.evalneg_ms += ms[3];
    c->acc.eval_batches += 1;
    c->acc.eval_pairs += pairs;
    c->acc.eval_groups += groups;
  }
}

extern "C" {

int w2v_set_timing(w2v_ctx *c, int on) {
  if (!c) return 1;
  if (on && !c->ev[0][0]) {
    for (int r = 0; r < kRing; r++)
      for (int k = 0; k < 5; k++) W2V_CHECK(cudaEventCreate(&c->ev[r][k]));
  }
  if (c->timing_on)
    for (int r = 0; r < kRing; r++) harvest(c, r);  // nothing of the old run leaks into the new one
  c->timing_on = on ? 1 : 0;
  for (int r = 0; r < kRing; r++) c->ev_state[r] = 0;
  memset(&c->acc, 0, sizeof(c->acc));
  return 0;
}

int w2v_get_timing(w2v_ctx *c, w2v_timing *out) {
  if (!c || !out) return 1;
  for (int r = 0; r < kRing; r++) harvest(c, r);
  *out = c->acc;
  return 0;
}

void w2v_default_opts(w2v_opts *o) {
  memset(o, 0, sizeof(*o));
  o->dim = 256;
  o->nskip = 5;
  o->nneg = 5;
  o->nreuse = 5;
  o->vocabSize = 100000;
  o->wexpt = 0.75f;
  o->wsample = 1e-4f;
  o->lrate = 1.0f;
  o->texp = 0.5f;
  o->vexp = 0.5f;
  o->iflip = 0;
  o->eqPosNeg = 0;
  o->permute = 0;
  o->seed = 0;
}

void w2v_destroy(w2v_ctx *c) {
  if (!c) return;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(c->device);
  cudaFree(c->tokens_in[1]);
  if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
  for (int k = 0; k < 2; k++) {
    if (c->ev_copied[k]) cudaEventDestroy(c->ev_copied[k]);
    if (c->ev_read[k]) cudaEventDestroy(c->ev_read[k]);
  }
  cudaFree(c->tokens); cudaFree(c->words); cudaFree(c->lb); cudaFree(c->ub); cudaFree(c->cnt);
  cudaFree(c->off); cudaFree(c->counts); cudaFree(c->ctx_in); cudaFree(c->ctx_out);
  cudaFree(c->wa); cudaFree(c->key_in); cudaFree(c->key_out); cudaFree(c->retvals);
  cudaFree(c->cub_tmp); cudaFree(c->hot_buf);
  cudaFreeHost(c->counts_host); cudaFreeHost(c->retvals_host);
  if (c->fault_host) cudaFreeHost(c->fault_host);
  for (int r = 0; r < kRing; r++)
    for (int k = 0; k < 5; k++) if (c->ev[r][k]) cudaEventDestroy(c->ev[r][k]);
  if (c->ev_counts) cudaEventDestroy(c->ev_counts);
  if (c->ev_pos) cudaEventDestroy(c->ev_pos);
  cudaSetDevice(prev);
  delete c;
}

int w2v_create(const w2v_opts *opts, int ncols, w2v_ctx **out) {
  if (!opts || !out || ncols <= 0) return 1;
  const w2v_opts &o = *opts;
  if (o.dim <= 0 || o.nskip < 1 || o.nskip > 15 || o.vocabSize <= 0 || o.nreuse < 1) return 1;
  if (!w2v::neg_shape_supported(o.nneg, o.nreuse)) {
    printf("word2vec unsupport size combination %d %d\n", o.nneg, o.nreuse);
    return 1;
  }
  w2v_ctx *c = new w2v_ctx();
  memset(c, 0, sizeof(*c));
  c->o = o;
  c->ncols = ncols;
  c->first_pos = -1;
  c->slice = w2v::whole_vocabulary();
  c->max_pairs = (int64_t)2 * o.nskip * ncols;
  if (c->max_pairs > 0x7fffffffLL) { delete c; return 1; }
  // expt and salpha exactly as Word2Vec.init forms them (Word2Vec.scala:139,150)
  c->expt = 1.0f / (1.0f - o.wexpt);
  c->salpha = o.wsample * (float)log((double)o.vocabSize);
  cudaError_t e = cudaGetDevice(&c->device);
  const size_t n4 = sizeof(int) * (size_t)ncols, p4 = sizeof(int) * (size_t)c->max_pairs;
  const int64_t max_groups = c->max_pairs / o.nreuse;
  size_t scan_bytes = 0, sort_bytes = 0;
  if (e == cudaSuccess) e = cudaMalloc(&c->tokens, 2 * n4);
  if (e == cudaSuccess) e = cudaMalloc(&c->tokens_in[1], 2 * n4);
  c->tokens_in[0] = c->tokens;
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking);
  for (int k = 0; k < 2 && e == cudaSuccess; k++) {
    e = cudaEventCreateWithFlags(&c->ev_copied[k], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_read[k], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaMalloc(&c->words, n4);
  if (e == cudaSuccess) e = cudaMalloc(&c->lb, n4);
  if (e == cudaSuccess) e = cudaMalloc(&c->ub, n4);
  if (e == cudaSuccess) e = cudaMalloc(&c->cnt, n4);
  if (e == cudaSuccess) e = cudaMalloc(&c->off, n4);
  if (e == cudaSuccess) e = cudaMalloc(&c->counts, 256);
  if (e == cudaSuccess) e = cudaMemset(c->counts, 0, 256);
  if (e == cudaSuccess) e = cudaHostAlloc(&c->fault_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) *c->fault_host = 0;
  if (e == cudaSuccess) e = cudaMalloc(&c->ctx_in, p4);
  if (e == cudaSuccess) e = cudaMalloc(&c->ctx_out, p4);
  if (e == cudaSuccess) e = cudaMalloc(&c->key_in, p4);
  if (e == cudaSuccess) e = cudaMalloc(&c->key_out, p4);
  if (e == cudaSuccess) e = cudaMalloc(&c->wa, sizeof(int) * (size_t)(max_groups + 1) * o.nneg);
  if (e == cudaSuccess) e = cudaMalloc(&c->retvals, 256);
  if (e == cudaSuccess && w2v::hot_levels_default() > 0) {
    e = cudaMalloc(&c->hot_buf, w2v::hot_rows_bytes());
    if (e == cudaSuccess) e = cudaMemset(c->hot_buf, 0, w2v::hot_rows_bytes());
  }
  c->hot = w2v::hot_rows_at(c->hot_buf, w2v::hot_levels_default());
  c->hot.stats = nullptr;   // set once the counts buffer exists
  if (e == cudaSuccess) e = cudaMallocHost(&c->counts_host, 256);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_counts, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_pos, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaMallocHost(&c->retvals_host, 256);
  if (e == cudaSuccess)
    e = cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, c->cnt, c->off, ncols);
  if (e == cudaSuccess)
    e = cub::DeviceRadixSort::SortPairsDescending(nullptr, sort_bytes, c->key_in, c->key_out,
                                                  c->ctx_in, c->ctx_out, (int)c->max_pairs, 0, 24);
  c->cub_tmp_bytes = (scan_bytes > sort_bytes ? scan_bytes : sort_bytes) + 256;
  if (e == cudaSuccess) e = cudaMalloc(&c->cub_tmp, c->cub_tmp_bytes);
  if (e != cudaSuccess) {
    w2v_destroy(c);
    return (int)e;
  }
  c->hot.stats = c->counts + 8;
  c->eval = reinterpret_cast<w2v::EvalScratch *>(c->counts + 32);
  *out = c;
  return 0;
}

int w2v_set_slice(w2v_ctx *c, int islice, int nslices, int nHead, int doHead) {
  if (!c || nslices < 1 || islice < 0 || islice >= nslices || nHead < 0) return 1;
  c->slice = w2v::SliceMap{nHead, nslices, islice, doHead};
  return 0;
}

int64_t w2v_slice_rows(int vocabSize, int nslices, int nHead) {
  // Word2Vec.init: nHeadTerms + 1 + (nfeats - nHeadTerms - 1) / nSlices (networks/Word2Vec.scala:106)
  if (nslices <= 1) return vocabSize;
  return (int64_t)nHead + 1 + (vocabSize - nHead - 1) / nslices;
}

int w2v_wait_pos(w2v_ctx *c, void *stream) {
  if (!c) return 1;
  if (!c->pos_recorded) return 0;
  return (int)cudaStreamWaitEvent((cudaStream_t)stream, c->ev_pos, 0);
}

int w2v_wait_before_neg(w2v_ctx *c, void *event) {
  if (!c) return 1;
  c->neg_wait = (cudaEvent_t)event;
  return 0;
}

int w2v_reserve_sms(w2v_ctx *c, int sms) {
  if (!c || sms < 0) return 1;
  c->sm_reserve = sms;
  return 0;
}

int w2v_apply_average(float *theta, const float *base, const float *avg, int64_t n, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n <= 0) return 0;
  if ((n & 3) || (((uintptr_t)theta | (uintptr_t)base | (uintptr_t)avg) & 15)) return 1;
  const int threads = 256;
  const int blocks = w2v::device_sm_count() * 8;
  w2v::apply_average_kernel<<<blocks, threads, 0, stream>>>(
      reinterpret_cast<float4 *>(theta), reinterpret_cast<const float4 *>(base),
      reinterpret_cast<const float4 *>(avg), n / 4);
  w2v::count_launch(1);
  return (int)cudaGetLastError();
}

int w2v_init_model(const w2v_opts *o, float *A, float *B, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const int64_t n = (int64_t)o->dim * o->vocabSize;
  W2V_CHECK(cudaMemsetAsync(A, 0, sizeof(float) * (size_t)n, stream));
  const int64_t blocks4 = (n + 3) / 4;
  const int threads = 256;
  w2v::init_model_kernel<<<(unsigned)((blocks4 + threads - 1) / threads), threads, 0, stream>>>(
      n, o->dim, make_rng(*o, 0), B);
  w2v::count_launch(1);
  return (int)cudaGetLastError();
}

static w2v::PermInverse invert(const w2v::PermKeys &k) {
  w2v::PermInverse inv;
  for (int r = 0; r < 4; r++) {
    // Newton's iteration for the inverse of an odd number modulo 2^32 (doubles the correct bits)
    uint32_t x = k.a[r];
    for (int it = 0; it < 5; it++) x *= 2u - k.a[r] * x;
    inv.ainv[r] = x;
    inv.c[r] = k.c[r];
  }
  return inv;
}

static w2v::PermKeys make_perm_keys(const w2v_opts &o, uint64_t batch_id);
static w2v::PermInverse make_perm_inverse(const w2v_opts &o, uint64_t batch_id) {
  return invert(make_perm_keys(o, batch_id));
}

static w2v::PermKeys make_perm_keys(const w2v_opts &o, uint64_t batch_id) {
  const w2v::Rng rng = make_rng(o, batch_id);
  const w2v::PhiloxOut x = w2v::philox4x32_10(0u, 0u, w2v::kStreamPermute, rng.batch, rng.k0, rng.k1);
  const w2v::PhiloxOut y = w2v::philox4x32_10(1u, 0u, w2v::kStreamPermute, rng.batch, rng.k0, rng.k1);
  w2v::PermKeys k;
  for (int r = 0; r < 4; r++) {
    k.a[r] = x.v[r] | 1u;
    k.c[r] = y.v[r];
  }
  return k;
}

// A staged kernel of an earlier minibatch gave up waiting for its copies (it dropped the
// rest of its columns): reported once, by the first call that finds the flag raised.
static int take_fault(w2v_ctx *c) {
  if (c->fault_host && *reinterpret_cast<volatile int *>(c->fault_host)) {
    *c->fault_host = 0;
    return (int)cudaErrorLaunchTimeout;
  }
  return 0;
}

// keep_list: also write the ordered pair list (w2v_buffers.contexts); the minibatch calls do not
// need it and build WB straight from the token windows.
static int wordmats(w2v_ctx *c, const int *tokens, const w2v_uniforms *u, uint64_t batch_id,
                    cudaStream_t stream, bool keep_list);

int w2v_wordmats(w2v_ctx *c, const int *tokens, const w2v_uniforms *u, uint64_t batch_id,
                 void *stream_) {
  return wordmats(c, tokens, u, batch_id, (cudaStream_t)stream_, true);
}

static int wordmats(w2v_ctx *c, const int *tokens, const w2v_uniforms *u, uint64_t batch_id,
                    cudaStream_t stream, bool keep_list) {
  Range range("w2v.wordmats");
  if (int fault = take_fault(c)) return fault;
  const w2v_opts &o = c->o;
  const int n = c->ncols;
  const int threads = 256, blocks = (n + threads - 1) / threads;
  const w2v::Rng rng = make_rng(o, batch_id);
  const float *us = u ? u->sample : nullptr, *uw = u ? u->window : nullptr;
  const float *up = u ? u->permute : nullptr, *un = u ? u->negs : nullptr;
  // permutation keys given by the caller can only be honoured by the sort
  const bool by_sort = (o.permute != 0) || (up != nullptr);

  c->slot = (int)(c->nbatch++ % kRing);
  c->ev_stream = stream;
  // the slot's events and counts are about to be overwritten: read them first
  // (waits for the batch that used the slot, kRing batches ago)
  if (c->timing_on) harvest(c, c->slot);
  c->ev_state[c->slot] = 0;
  mark(c, 0, stream);
  W2V_CHECK(cudaMemsetAsync(c->counts + 8, 0, 2 * sizeof(int), stream));   // the hot-word statistics
  w2v::words_bounds_kernel<<<blocks, threads, 0, stream>>>(
      n, tokens, o.iflip ? 1 : 0, o.vocabSize, o.nskip, c->salpha, us, uw, rng, c->words, c->lb, c->ub,
      c->counts + 8);
  w2v::count_pairs_kernel<<<blocks, threads, 0, stream>>>(n, c->words, c->lb, c->ub, c->cnt);
  size_t tmp = c->cub_tmp_bytes;
  W2V_CHECK(cub::DeviceScan::ExclusiveSum(c->cub_tmp, tmp, c->cnt, c->off, n, stream));
  w2v::totals_kernel<<<1, 32, 0, stream>>>(n, c->cnt, c->off, o.nreuse, c->counts);
  W2V_CHECK(cudaMemcpyAsync(c->counts_host + 2 * c->slot, c->counts, 2 * sizeof(int),
                            cudaMemcpyDeviceToHost, stream));
  W2V_CHECK(cudaEventRecord(c->ev_counts, stream));
  c->counts_pending = 1;
  keep_list = keep_list || by_sort;
  c->have_list = keep_list ? 1 : 0;
  if (keep_list)
    w2v::fill_pairs_kernel<<<blocks, threads, 0, stream>>>(n, o.nskip, c->words, c->lb, c->ub, c->off,
                                                          up, rng, c->ctx_in,
                                                          by_sort ? c->key_in : nullptr);
  w2v::count_launch(keep_list ? 4 : 3);
  W2V_CHECK(cudaGetLastError());
  mark(c, 1, stream);
  if (by_sort) {
    // the sort needs the pair count on the host
    int err = settle_counts(c);
    if (err) return err;
    if (c->npairs > 0) {
      tmp = c->cub_tmp_bytes;
      W2V_CHECK(cub::DeviceRadixSort::SortPairsDescending(c->cub_tmp, tmp, c->key_in, c->key_out,
                                                          c->ctx_in, c->ctx_out, (int)c->npairs, 0,
                                                          24, stream));
    }
    const int64_t nn = (int64_t)c->ngroups * o.nneg;
    if (nn > 0) {
      w2v::negative_ids_kernel<<<(unsigned)((nn + threads - 1) / threads), threads, 0, stream>>>(
          nn, nullptr, o.nneg, un, rng, o.vocabSize, c->expt, c->wa);
      w2v::count_launch(1);
    }
  } else {
    // everything downstream reads the counts on the device: nothing waits for the host
    const int64_t max_groups = c->max_pairs / o.nreuse;
    const int64_t max_negs = max_groups * o.nneg;
    if (!keep_list && c->max_pairs > 0) {
      w2v::scatter_pairs_kernel<<<blocks, threads, 0, stream>>>(
          n, c->counts, o.nreuse, make_perm_inverse(o, batch_id), c->words, c->lb, c->ub, c->off, c->ctx_out);
      w2v::count_launch(1);
    } else if (c->max_pairs > 0) {
      const int shuffle_blocks = (int)std::min<int64_t>((c->max_pairs + threads - 1) / threads,
                                                       (int64_t)w2v::device_sm_count() * 16);
      w2v::shuffle_contexts_kernel<<<shuffle_blocks, threads, 0, stream>>>(
          c->counts, o.nreuse, make_perm_keys(o, batch_id), c->ctx_in, c->ctx_out);
      w2v::count_launch(1);
    }
    if (max_negs > 0) {
      w2v::negative_ids_kernel<<<(unsigned)((max_negs + threads - 1) / threads), threads, 0, stream>>>(
          max_negs, c->counts, o.nneg, un, rng, o.vocabSize, c->expt, c->wa);
      w2v::count_launch(1);
    }
  }
  mark(c, 2, stream);
  return (int)cudaGetLastError();
}

int w2v_buffers(w2v_ctx *c, w2v_buffers_t *out) {
  if (!c || !out) return 1;
  int err = settle_counts(c);
  if (err) return err;
  out->words = c->words; out->lb = c->lb; out->ub = c->ub;
  out->contexts = c->have_list ? c->ctx_in : nullptr;
  out->WB = c->ctx_out;
  out->WA = c->wa;
  out->npairs = c->npairs;
  out->ngroups = c->ngroups;
  return 0;
}

// Column count of the negative kernels: known on the host after a sort, else
// an upper bound for the grid plus the device-side count.
static void group_count(const w2v_ctx *c, int *ncols, const int **ncols_dev) {
  if (c->counts_pending) {
    *ncols = (int)(c->max_pairs / c->o.nreuse);
    *ncols_dev = c->counts + 1;
  } else {
    *ncols = c->ngroups;
    *ncols_dev = nullptr;
  }
}

int w2v_dobatch(w2v_ctx *c, const int *tokens, const w2v_uniforms *u, float *A, float *B,
                int64_t pos, uint64_t batch_id, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const w2v_opts &o = c->o;
  // learning-rate schedule of Word2Vec.dobatch (Word2Vec.scala:170-177)
  if (c->first_pos < 0) c->first_pos = pos;
  const float nsteps = (float)pos / (float)c->first_pos;
  const float lrpos = o.lrate * (float)pow((double)nsteps, -(double)o.texp);
  const float lrneg = o.eqPosNeg ? lrpos : lrpos / (float)o.nneg;
  int err = wordmats(c, tokens, u, batch_id, stream, false);
  if (err) return err;
  {
    Range range("w2v.pos");
    err = w2v::pos_update_async(o.dim, c->ncols, nullptr, o.nskip, c->words, c->lb, c->ub, A, B,
                                lrpos, o.vexp, c->hot, c->slice, stream);
  }
  if (err) return err;
  W2V_CHECK(cudaEventRecord(c->ev_pos, stream));
  c->pos_recorded = 1;
  mark(c, 3, stream);
  if (c->neg_wait) {
    W2V_CHECK(cudaStreamWaitEvent(stream, c->neg_wait, 0));
    c->neg_wait = nullptr;
  }
  w2v::SmReserve reserve(c->sm_reserve);   // the negative update leaves these SMs to another stream's kernel
  int groups = 0;
  const int *groups_dev = nullptr;
  group_count(c, &groups, &groups_dev);
  {
    Range range("w2v.neg");
    err = w2v::neg_update_async(o.dim, groups, groups_dev, 0x7fffffff, o.nneg, o.nreuse, c->wa,
                                c->ctx_out, A, B, lrneg, o.vexp, c->hot, c->fault_host, c->slice, stream);
  }
  mark(c, 4, stream);
  if (c->timing_on) c->ev_state[c->slot] = 1;
  return err;
}

int w2v_evalbatch(w2v_ctx *c, const int *tokens, const w2v_uniforms *u, const float *A,
                  const float *B, uint64_t batch_id, double *score_host, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const w2v_opts &o = c->o;
  int err = wordmats(c, tokens, u, batch_id, stream, false);
  if (err) return err;
  W2V_CHECK(cudaMemsetAsync(c->retvals, 0, 2 * sizeof(float), stream));
  {
    Range range("w2v.evalpos");
    err = w2v::pos_eval_async(o.dim, c->ncols, nullptr, o.nskip, c->words, c->lb, c->ub, A, B,
                              c->retvals, c->eval, c->slice, stream);
  }
  if (err) return err;
  mark(c, 3, stream);
  int groups = 0;
  const int *groups_dev = nullptr;
  group_count(c, &groups, &groups_dev);
  {
    Range range("w2v.evalneg");
    err = w2v::neg_eval_async(o.dim, groups, groups_dev, o.nneg, o.nreuse, c->wa, c->ctx_out, A, B,
                              c->retvals + 1, c->eval, c->fault_host, c->slice, stream);
  }
  if (err) return err;
  mark(c, 4, stream);
  if (c->timing_on) c->ev_state[c->slot] = 2;
  W2V_CHECK(cudaMemcpyAsync(c->retvals_host, c->retvals, 2 * sizeof(float), cudaMemcpyDeviceToHost, stream));
  W2V_CHECK(cudaStreamSynchronize(stream));
  err = settle_counts(c);
  if (err) return err;
  err = take_fault(c);
  if (err) return err;
  const double epos = c->retvals_host[0], eneg = c->retvals_host[1];
  const double denom = (double)c->ngroups * o.nreuse;
  // (epos + eneg / nneg) / goodwords.length  (Word2Vec.scala:209)
  *score_host = denom > 0 ? (epos + eneg / (o.eqPosNeg ? 1 : o.nneg)) / denom : 0.0;
  return 0;
}

// Uploads a host minibatch into the token buffer whose turn it is, on the copy
// stream, and makes `stream` wait for it.  The buffer was last read by the
// preprocessing of the call before the previous one.
static int upload_tokens(w2v_ctx *c, const int *tokens_host, cudaStream_t stream, int **dev, int *which) {
  const int k = (int)(c->host_calls++ & 1);
  *which = k;
  if (c->read_recorded[k]) W2V_CHECK(cudaStreamWaitEvent(c->copy_stream, c->ev_read[k], 0));
  W2V_CHECK(cudaMemcpyAsync(c->tokens_in[k], tokens_host, 2 * sizeof(int) * (size_t)c->ncols,
                            cudaMemcpyHostToDevice, c->copy_stream));
  W2V_CHECK(cudaEventRecord(c->ev_copied[k], c->copy_stream));
  W2V_CHECK(cudaStreamWaitEvent(stream, c->ev_copied[k], 0));
  *dev = c->tokens_in[k];
  return 0;
}

int w2v_dobatch_host(w2v_ctx *c, const int *tokens_host, float *A, float *B, int64_t pos,
                     uint64_t batch_id, int64_t *npairs_host, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int *dev = nullptr;
  int k = 0;
  int err = upload_tokens(c, tokens_host, stream, &dev, &k);
  if (err) return err;
  err = w2v_dobatch(c, dev, nullptr, A, B, pos, batch_id, stream);
  if (err) return err;
  // only the preprocessing reads the tokens; it is enqueued ahead of the update kernels,
  // but an event recorded here completes after them: good enough two calls later
  W2V_CHECK(cudaEventRecord(c->ev_read[k], stream));
  c->read_recorded[k] = 1;
  // the pair count is this call's result: wait for it (and thereby for the upload, so the
  // caller may reuse its host buffer), not for the update kernels, which finish in stream order
  err = settle_counts(c);
  if (err) return err;
  if (npairs_host) *npairs_host = c->npairs;
  return (int)cudaGetLastError();
}

int w2v_evalbatch_host(w2v_ctx *c, const int *tokens_host, const float *A, const float *B,
                       uint64_t batch_id, double *score_host, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int *dev = nullptr;
  int k = 0;
  int err = upload_tokens(c, tokens_host, stream, &dev, &k);
  if (err) return err;
  err = w2v_evalbatch(c, dev, nullptr, A, B, batch_id, score_host, stream);  // synchronises
  if (err) return err;
  W2V_CHECK(cudaEventRecord(c->ev_read[k], stream));
  c->read_recorded[k] = 1;
  return 0;
}

}  // extern "C"
