// Device-side building blocks shared by the Word2Vec SGNS kernels (sm_100a).
//
// A model matrix is column-major dim x vocab fp32, so word `w` is the
// contiguous row `[w*dim, (w+1)*dim)`.  A warp owns a row at a time: lane `l`
// holds the 16-byte vectors `l, l+32, l+64, ...` of the row, which makes every
// row load and every row update a fully coalesced 128-bit access.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace w2v {

constexpr unsigned kFullMask = 0xffffffffu;

// Logistic function with the reference's guards: above 16 it is exactly 1,
// below -16 exactly 0 (jni/src/DNN127.cu:128-135, BIDMach_CPUMACH.c:48-55).
// expf and the division are the IEEE-accurate versions (no fast-math), so the
// result tracks the CPU path to a few ulp.
__device__ __forceinline__ float sigmoid_guard(float x) {
  if (x > 16.0f) return 1.0f;
  if (x < -16.0f) return 0.0f;
  float e = expf(x);
  return e / (1.0f + e);
}

// log(max(v, 1e-20)) of one pair's probability, evaluated in fp32 as the
// reference kernels do (jni/src/DNN127.cu:318); the sums are kept in double.
__device__ __forceinline__ double pair_score(float v) { return (double)logf(fmaxf(v, 1.0e-20f)); }

// (1 + id)^vexp, the per-word learning-rate scale (BIDMach_CPUMACH.c:33,42;
// jni/src/DNN127.cu:145,149 forms the same value from the row offset).
__device__ __forceinline__ float freq_scale(int id, float vexp) {
  if (vexp == 0.0f) return 1.0f;
  if (vexp == 0.5f) return sqrtf((float)(1 + id));  // the reference's default exponent
  if (vexp == 1.0f) return (float)(1 + id);
  return powf((float)(1 + id), vexp);
}

// 128-bit fire-and-forget atomic add into global memory (one L2 reduction per
// 16 bytes instead of four scalar atomics).
__device__ __forceinline__ void red_add_v4(float *addr, float4 v) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFullMask, v, off);
  return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFullMask, v, off);
  return v;
}

// Row held in registers: NR vectors of 4 floats per lane.
template <int NR>
struct Row {
  float4 v[NR];
};

template <int NR>
__device__ __forceinline__ void row_zero(Row<NR> &r) {
#pragma unroll
  for (int q = 0; q < NR; q++) r.v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// Load row `w` (w >= 0) of a dim x vocab matrix.  nvec = dim / 4.
template <int NR>
__device__ __forceinline__ void row_load(Row<NR> &r, const float *M, int64_t w, int dim, int nvec,
                                         int lane) {
  const float4 *p = reinterpret_cast<const float4 *>(M + w * (int64_t)dim);
#pragma unroll
  for (int q = 0; q < NR; q++) {
    int idx = lane + 32 * q;
    r.v[q] = (idx < nvec) ? p[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <int NR>
__device__ __forceinline__ float row_dot_partial(const Row<NR> &a, const Row<NR> &b) {
  float s = 0.f;
#pragma unroll
  for (int q = 0; q < NR; q++) {
    s = fmaf(a.v[q].x, b.v[q].x, s);
    s = fmaf(a.v[q].y, b.v[q].y, s);
    s = fmaf(a.v[q].z, b.v[q].z, s);
    s = fmaf(a.v[q].w, b.v[q].w, s);
  }
  return s;
}

// acc += c * x
template <int NR>
__device__ __forceinline__ void row_axpy(Row<NR> &acc, float c, const Row<NR> &x) {
#pragma unroll
  for (int q = 0; q < NR; q++) {
    acc.v[q].x = fmaf(c, x.v[q].x, acc.v[q].x);
    acc.v[q].y = fmaf(c, x.v[q].y, acc.v[q].y);
    acc.v[q].z = fmaf(c, x.v[q].z, acc.v[q].z);
    acc.v[q].w = fmaf(c, x.v[q].w, acc.v[q].w);
  }
}

// ---------------------------------------------------------------------------
// Many-value warp reduction.  Each lane brings M partial sums; five exchange
// steps later the M totals are spread over the lanes (FIN per lane) instead of
// every lane holding every total, which takes about M shuffles rather than
// 5*M, and lets the sigmoid of each total be evaluated by one lane only.
// Total `idx` ends up in slot slot_of(idx) of lane lane_of(idx).
// ---------------------------------------------------------------------------
template <int M>
struct Spread {
  static constexpr int h1 = (M + 1) / 2, h2 = (h1 + 1) / 2, h3 = (h2 + 1) / 2, h4 = (h3 + 1) / 2,
                       h5 = (h4 + 1) / 2;
  static constexpr int FIN = h5;

  static __host__ __device__ constexpr int lane_of(int idx) {
    int lane = 0;
    const int hs[5] = {h1, h2, h3, h4, h5};
    for (int s = 0; s < 5; s++) {
      if (idx >= hs[s]) {
        lane |= (16 >> s);
        idx -= hs[s];
      }
    }
    return lane;
  }
  static __host__ __device__ constexpr int slot_of(int idx) {
    const int hs[5] = {h1, h2, h3, h4, h5};
    for (int s = 0; s < 5; s++)
      if (idx >= hs[s]) idx -= hs[s];
    return idx;
  }

  template <int CUR, int OFF>
  static __device__ __forceinline__ void step(float (&v)[M], int lane) {
    constexpr int H = (CUR + 1) / 2;
    const bool up = (lane & OFF) != 0;
#pragma unroll
    for (int i = 0; i < H; i++) {
      float lo = v[i];
      float hi = (i + H < CUR) ? v[i + H] : 0.f;
      float send = up ? lo : hi;
      float keep = up ? hi : lo;
      v[i] = keep + __shfl_xor_sync(kFullMask, send, OFF);
    }
  }

  static __device__ __forceinline__ void reduce(float (&v)[M], int lane) {
    step<M, 16>(v, lane);
    step<h1, 8>(v, lane);
    step<h2, 4>(v, lane);
    step<h3, 2>(v, lane);
    step<h4, 1>(v, lane);
  }
};

// Which lanes hold a real total in slot q after Spread<M>::reduce.
template <int M>
__host__ __device__ constexpr unsigned spread_valid_mask(int q) {
  unsigned m = 0;
  for (int idx = 0; idx < M; idx++)
    if (Spread<M>::slot_of(idx) == q) m |= 1u << Spread<M>::lane_of(idx);
  return m;
}

// Calls f(integral_constant<q>) on every lane that holds a real total in slot
// q after Spread<M>::reduce.  The masks are constant expressions: left to the
// optimiser, the loops of lane_of / slot_of were seen to survive into the kernel.
template <int M, int Q = 0, class F>
__device__ __forceinline__ void for_valid_totals(int lane, F &&f) {
  if constexpr (Q < Spread<M>::FIN) {
    constexpr unsigned valid = spread_valid_mask<M>(Q);
    if ((valid >> lane) & 1u) f(std::integral_constant<int, Q>());
    for_valid_totals<M, Q + 1>(lane, f);
  }
}

// g[idx] = total idx of a Spread<M>::reduce, on every lane; source lane and
// slot are constant expressions.
template <int M, int I = 0>
__device__ __forceinline__ void broadcast_totals(const float (&p)[M], float (&g)[M]) {
  if constexpr (I < M) {
    constexpr int src_lane = Spread<M>::lane_of(I), slot = Spread<M>::slot_of(I);
    g[I] = __shfl_sync(kFullMask, p[slot], src_lane);
    broadcast_totals<M, I + 1>(p, g);
  }
}

// Lane l < NWA carries A-word l of the column, lanes NWA..NWA+NWB-1 the
// B-words.  Ids at or above `nwords` are masked to -1 (word2vecNegFilt,
// jni/src/DNN127.cu:690-712): a masked word acts as a zero row and is not
// updated.
template <int NWA, int NWB>
__device__ __forceinline__ int column_word(const int *__restrict__ WA, const int *__restrict__ WB,
                                           int64_t col, int nwords, int lane) {
  int w = -1;
  if (lane < NWA)
    w = WA[col * NWA + lane];
  else if (lane < NWA + NWB)
    w = WB[col * NWB + (lane - NWA)];
  if (w >= nwords) w = -1;
  return w;
}

template <int NWA, int NWB, int NR>
__device__ __forceinline__ void column_dots(const Row<NR> (&a)[NWA], const Row<NR> (&b)[NWB],
                                            float (&p)[NWA * NWB], int lane) {
#pragma unroll
  for (int j = 0; j < NWA; j++)
#pragma unroll
    for (int k = 0; k < NWB; k++) p[j * NWB + k] = row_dot_partial(a[j], b[k]);
  Spread<NWA * NWB>::reduce(p, lane);
}

// ---------------------------------------------------------------------------
// Packed fp32x2 arithmetic (sm_100 executes two fp32 FMAs per instruction on a
// 64-bit register pair) and rows held as such pairs.
// ---------------------------------------------------------------------------
typedef unsigned long long u64;

__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
  u64 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
  u64 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 pack2(float x, float y) {
  u64 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(x), "f"(y));
  return d;
}
__device__ __forceinline__ void unpack2(u64 v, float &x, float &y) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}

template <int NR>
struct PRow {
  u64 v[NR][2];  // vector q of the lane = {v[q][0], v[q][1]} = 4 floats
};

template <int NR>
__device__ __forceinline__ void prow_zero(PRow<NR> &r) {
#pragma unroll
  for (int q = 0; q < NR; q++) r.v[q][0] = r.v[q][1] = 0ull;
}

template <int NR>
__device__ __forceinline__ float prow_dot_partial(const PRow<NR> &a, const PRow<NR> &b) {
  // one packed accumulator: many dot products are always in flight, so the
  // longer dependency chain costs nothing and the final sum is one add
  u64 s = mul2(a.v[0][0], b.v[0][0]);
  s = fma2(a.v[0][1], b.v[0][1], s);
#pragma unroll
  for (int q = 1; q < NR; q++) {
    s = fma2(a.v[q][0], b.v[q][0], s);
    s = fma2(a.v[q][1], b.v[q][1], s);
  }
  float x, y;
  unpack2(s, x, y);
  return x + y;
}

// acc = c * x
template <int NR>
__device__ __forceinline__ void prow_scale(PRow<NR> &acc, float c, const PRow<NR> &x) {
  const u64 cc = pack2(c, c);
#pragma unroll
  for (int q = 0; q < NR; q++) {
    acc.v[q][0] = mul2(cc, x.v[q][0]);
    acc.v[q][1] = mul2(cc, x.v[q][1]);
  }
}

// acc += c * x
template <int NR>
__device__ __forceinline__ void prow_axpy(PRow<NR> &acc, float c, const PRow<NR> &x) {
  const u64 cc = pack2(c, c);
#pragma unroll
  for (int q = 0; q < NR; q++) {
    acc.v[q][0] = fma2(cc, x.v[q][0], acc.v[q][0]);
    acc.v[q][1] = fma2(cc, x.v[q][1], acc.v[q][1]);
  }
}

// ---------------------------------------------------------------------------
// Bulk asynchronous copies (TMA, untiled form) global -> shared, completion
// signalled on an mbarrier in shared memory.  Addresses and sizes must be
// multiples of 16 bytes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_addr(const void *p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(u64 *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(u64 *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u64 *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity, giving up after `limit` polls.
__device__ __forceinline__ bool mbar_wait_bounded(u64 *bar, unsigned parity, int limit) {
  for (int spins = 0; spins < limit; spins++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_load_row(void *smem_dst, const void *gsrc, unsigned bytes,
                                              u64 *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void async_proxy_fence() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Bulk reduction shared -> global: adds `bytes` / 4 floats at smem_src to those at gdst
// (both 16-byte aligned, bytes a multiple of 16).  Completion through bulk groups.
__device__ __forceinline__ void bulk_reduce_add_row(float *gdst, const void *smem_src, unsigned bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_group_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

}  // namespace w2v
