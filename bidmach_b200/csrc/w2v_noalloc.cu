// word2vecEvalNegNoAlloc: the negative-pair scoring kernel for hosts that must
// not allocate device memory.
//
// Who needs it.  BIDMach runs inside a JVM whose matrix library (BIDMat) keeps
// its own device-memory cache and is routinely sized to fill the card, so a
// cudaMalloc issued by a native library in the middle of a run can fail or
// take memory the cache counted on.  The same holds for serving processes that
// freeze their memory map after warm-up.  The regular scoring entry points
// borrow a small accumulator from a pool that grows with cudaMalloc when every
// set is in use; this one takes none: its scratch memory is a fixed array
// compiled into the library's device image.
//
// What that costs.  The array (kScratchBytes, about 64 KiB) exists on every GPU
// that loads the library, for the life of the process, whether or not this
// entry point is ever called.  Its size bounds the input: one partial sum per
// block of kColsPerBlock columns, kMaxBlocks partial sums, so at most
// kMaxCols = kMaxBlocks * kColsPerBlock columns per call; more is refused.
// All calls on a device share the array, and it still holds what the previous
// call left there: the arrival counter is cleared at the start of every call,
// and every partial-sum slot that is read has been overwritten by this call
// first.  Two calls that are in flight on the same GPU at the same time (from
// different streams or threads) would overwrite each other's partial sums:
// callers must not overlap them.
//
// Set-up.  In host code the array's name is only a handle; the device address
// that a kernel can use comes from cudaGetSymbolAddress, once per device, with
// that device current.  The first call on each device does this; it should come
// before the process starts any stream capture on that device.  Like the
// other launchers the function runs on the calling thread's default stream and
// waits for the kernel before it returns.
//
// Results.  Each block sums its own columns in double; the block that finishes
// last adds the partial sums in slot order, so the total does not depend on
// the order in which blocks finish.  It equals word2vecEvalNeg's up to the
// order of double additions; a negative word id counts as a zero row, as there.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "w2v_device.cuh"
#include "w2v_internal.h"

namespace {

constexpr int kThreads = 128;
constexpr int kColsPerBlock = 256;
constexpr int kMaxBlocks = 8192;
constexpr int kMaxCols = kMaxBlocks * kColsPerBlock;  // 2,097,152 columns per call
constexpr int kHeaderBytes = 256;
constexpr size_t kScratchBytes = kHeaderBytes + sizeof(double) * kMaxBlocks;

// [0,4): arrival counter; [256, ...): one double per block
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

template <int NWA, int NWB>
__global__ void __launch_bounds__(kThreads)
    eval_neg_static_kernel(int dim, int ncols, const int *__restrict__ WA,
                           const int *__restrict__ WB, const float *__restrict__ A,
                           const float *__restrict__ B, unsigned char *scratch, float *retval) {
  using namespace w2v;
  using S = Spread<NWA * NWB>;
  unsigned *arrived = reinterpret_cast<unsigned *>(scratch);
  double *partial = reinterpret_cast<double *>(scratch + kHeaderBytes);
  __shared__ double warp_part[kThreads / 32];
  __shared__ bool is_last;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int first = blockIdx.x * kColsPerBlock;
  const int last = min(ncols, first + kColsPerBlock);
  double acc = 0.0;
  for (int col = first + warp; col < last; col += kThreads / 32) {
    const int myw = column_word<NWA, NWB>(WA, WB, col, 0x7fffffff, lane);
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
    for_valid_totals<NWA * NWB>(
        lane, [&](auto q) { acc += pair_score(1.0f - sigmoid_guard(p[decltype(q)::value])); });
  }

  acc = warp_sum(acc);
  if (lane == 0) warp_part[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int k = 0; k < kThreads / 32; k++) tot += warp_part[k];
    partial[blockIdx.x] = tot;
    __threadfence();
    is_last = (atomicAdd(arrived, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last && warp == 0) {
    __threadfence();
    const volatile double *vp = partial;
    double tot = 0;
    for (int k = lane; k < (int)gridDim.x; k += 32) tot += vp[k];
    tot = warp_sum(tot);
    if (lane == 0) {
      atomicAdd(retval, (float)tot);
      *arrived = 0u;
    }
  }
}

// Device address of g_scratch on the current device, looked up once per device.
int scratch_address(unsigned char **out) {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static unsigned char *per_dev[kMaxDev] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDev) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!per_dev[dev]) {
    unsigned char *p = nullptr;
    e = cudaGetSymbolAddress((void **)&p, g_scratch);
    if (e != cudaSuccess) return (int)e;
    per_dev[dev] = p;
  }
  *out = per_dev[dev];
  return 0;
}

template <int NWA, int NWB>
int launch(int dim, int ncols, const int *WA, const int *WB, const float *A, const float *B,
           unsigned char *scratch, float *retval, cudaStream_t stream) {
  const int blocks = (ncols + kColsPerBlock - 1) / kColsPerBlock;
  eval_neg_static_kernel<NWA, NWB><<<blocks, kThreads, 0, stream>>>(dim, ncols, WA, WB, A, B,
                                                                    scratch, retval);
  w2v::count_launch(1);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" int word2vecEvalNegNoAlloc(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB,
                                      float *A, float *B, float *Retval) {
  if (!w2v::neg_shape_supported(nwa, nwb)) {
    printf("word2vecEvalNegNoAlloc unsupport size combination %d %d\n", nwa, nwb);
    return 1;
  }
  if (ncols > kMaxCols) {
    printf("word2vecEvalNegNoAlloc: %d columns exceed the built-in scratch array's limit of %d; "
           "split the call or use word2vecEvalNeg\n", ncols, kMaxCols);
    return 1;
  }
  if (ncols <= 0) return 0;
  if (nrows <= 0) return 1;
  unsigned char *scratch = nullptr;
  int err = scratch_address(&scratch);
  if (err) return err;
  cudaStream_t stream = cudaStreamPerThread;
  cudaError_t e = cudaMemsetAsync(scratch, 0, kHeaderBytes, stream);
  if (e != cudaSuccess) return (int)e;
  switch (nwa * 10000 + nwb) {
    case 50001: err = launch<5, 1>(nrows, ncols, WA, WB, A, B, scratch, Retval, stream); break;
    case 50005: err = launch<5, 5>(nrows, ncols, WA, WB, A, B, scratch, Retval, stream); break;
    case 100005: err = launch<10, 5>(nrows, ncols, WA, WB, A, B, scratch, Retval, stream); break;
    default: err = launch<5, 10>(nrows, ncols, WA, WB, A, B, scratch, Retval, stream); break;
  }
  if (err) return err;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
