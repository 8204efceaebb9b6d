// Row-traffic probe, a measuring aid of the benchmark and not part of the C-ABI
// library: it is built into a library of its own (libw2vrowprobe.so) that only
// bench.py loads.
//
// It runs the memory side of the negative update or of the negative scoring
// with the arithmetic left out, on the columns it is given.  Mode 0 adds a row
// of zeros to every row of every column with the update kernel's 16-byte atomic
// reductions, hot ids going to replica rows as in the update kernel (the model
// keeps its values); mode 1 reads every row; mode 2 does both as the update
// kernel does, a column's rows read first and the zeros added afterwards (the
// reductions then find their rows in the L2, which they do not in mode 0).  The
// duration of the launch is what the memory system alone needs for the scatter,
// the gather, or the gather and scatter of one negative update (scoring) launch.
#include <cuda_runtime.h>
#include <stdint.h>

#include "w2v_rows.cuh"

namespace {

using namespace w2v;

constexpr int kLevels = 4, kReps = 16, kMaxDim = 1280;   // the update kernels' defaults

template <int NR, int MODE>
__global__ void __launch_bounds__(512) row_probe_kernel(int dim, int ncols, int nwa, int nwb,
                                                        const int *__restrict__ WA,
                                                        const int *__restrict__ WB, float *A, float *B,
                                                        HotRows hot, float *sink) {
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 2;
  const bool tail = lane + 32 * (NR - 1) < nvec;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  PRow<NR> zero;
  prow_zero(zero);
  float seen = 0.f;
  for (int col = gwarp; col < ncols; col += nwarps) {
    int myw = 0;
    if (lane < nwa)
      myw = WA[(int64_t)col * nwa + lane];
    else if (lane < nwa + nwb)
      myw = WB[(int64_t)col * nwb + (lane - nwa)];
    for (int r = 0; MODE != 2 && r < nwa + nwb; r++) {
      const int w = __shfl_sync(kFullMask, myw, r);
      if (w < 0) continue;
      if (MODE == 0) {
        float *dst = (r < nwa) ? update_target(A, hot.shadowA, hot, w, dim, gwarp)
                               : update_target(B, hot.shadowB, hot, w, dim, gwarp);
        prow_red_lane(dst + 4 * lane, tail, zero);
      } else if (MODE == 1) {
        PRow<NR> row;
        prow_load_lane(row, reinterpret_cast<const ulonglong2 *>((r < nwa ? A : B) + (int64_t)w * dim) + lane,
                       tail);
        seen += prow_dot_partial(row, row);
      }
    }
    if (MODE == 2) {
      // as many rows in flight at a time as the registers hold
      constexpr int CH = NR <= 4 ? 5 : (NR <= 8 ? 2 : 1);
      for (int r0 = 0; r0 < nwa + nwb; r0 += CH) {
        PRow<NR> rows[CH];
        int ws[CH];
#pragma unroll
        for (int k = 0; k < CH; k++) {
          const int w = __shfl_sync(kFullMask, myw, (r0 + k) & 31);
          ws[k] = (r0 + k < nwa + nwb) ? w : -1;
          prow_zero(rows[k]);
          if (ws[k] >= 0)
            prow_load_lane(rows[k],
                           reinterpret_cast<const ulonglong2 *>((r0 + k < nwa ? A : B) + (int64_t)ws[k] * dim) + lane,
                           tail);
        }
#pragma unroll
        for (int k = 0; k < CH; k++) {
          if (ws[k] < 0) continue;
          seen += prow_dot_partial(rows[k], rows[k]);
          float *dst = (r0 + k < nwa) ? update_target(A, hot.shadowA, hot, ws[k], dim, gwarp)
                                      : update_target(B, hot.shadowB, hot, ws[k], dim, gwarp);
          prow_red_lane(dst + 4 * lane, tail, zero);
        }
      }
    }
  }
  if (MODE != 0 && seen == -1.0f) *sink = seen;  // keeps the loads alive; never true
}

float *g_buf = nullptr;   // replica rows + one float; single device, single thread (the benchmark)

}  // namespace

extern "C" int w2v_rowprobe(int dim, int ncols, int nwa, int nwb, const int *WA, const int *WB, float *A,
                            float *B, int mode, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (ncols <= 0) return 0;
  if (dim <= 0 || (dim & 3) || dim > kMaxDim || nwa + nwb > 32 || mode < 0 || mode > 2) return 1;
  const size_t rows = (size_t)kLevels * kReps;
  if (!g_buf) {
    const size_t bytes = sizeof(float) * (2 * rows * kMaxDim + 4);
    cudaError_t e = cudaMalloc(&g_buf, bytes);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(g_buf, 0, bytes);
    if (e != cudaSuccess) return (int)e;
  }
  HotRows hot;
  hot.shadowA = g_buf;
  hot.shadowB = g_buf + rows * kMaxDim;
  hot.limit = 1 << kLevels;
  hot.rmax = kReps;
  hot.fold_every = 0;
  hot.stats = nullptr;
  float *sink = g_buf + 2 * rows * kMaxDim;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = sms * 8;
  const int nr = (dim / 4 + 31) / 32;
#define PROBE_CASE(NRV)                                                                                       \
  case NRV:                                                                                                   \
    if (mode == 0)                                                                                            \
      row_probe_kernel<NRV, 0><<<grid, 512, 0, stream>>>(dim, ncols, nwa, nwb, WA, WB, A, B, hot, sink);       \
    else if (mode == 1)                                                                                       \
      row_probe_kernel<NRV, 1><<<grid, 512, 0, stream>>>(dim, ncols, nwa, nwb, WA, WB, A, B, hot, sink);       \
    else                                                                                                      \
      row_probe_kernel<NRV, 2><<<grid, 512, 0, stream>>>(dim, ncols, nwa, nwb, WA, WB, A, B, hot, sink);       \
    break;
  switch (nr) {
    PROBE_CASE(1) PROBE_CASE(2) PROBE_CASE(3) PROBE_CASE(4) PROBE_CASE(5) PROBE_CASE(6) PROBE_CASE(7)
    PROBE_CASE(8) PROBE_CASE(9) PROBE_CASE(10)
    default: return 1;
  }
#undef PROBE_CASE
  return (int)cudaGetLastError();
}
