// Model exchange between replicas: the replacement of Word2Vec.mergeModelFn
// (networks/Word2Vec.scala:547-568), which averages the model matrices of all
// GPUs through host-driven peer copies.  Two forms:
//
// 1. w2v_nvls_average: one kernel per replica that averages a buffer mapped on
//    every GPU through an NVLink multicast address.  Replica r owns the r-th
//    slice of the buffer: a `multimem.ld_reduce` fetches the sum over all
//    replicas of 16 bytes (the NVSwitch adds them on the way), the kernel scales
//    it by 1 / replicas and a `multimem.st` writes the mean back into every
//    replica.  Every GPU therefore sends and receives the buffer once, and the
//    kernel holds no data and waits for nobody: it can run beside the update
//    kernels of the next minibatch on a few SMs.  The buffer must have been
//    allocated as symmetric memory with a multicast mapping (one process per GPU;
//    torch.distributed's symmetric memory does that).
//
//    w2v_p2p_average does the same with plain loads and stores on the replicas' own addresses
//    of the buffer (every replica reads its slice from all peers, adds, and writes the mean to
//    all of them).  A multimem access moves the requester's own copy through the switch as well,
//    n * (1 + 1/replicas) bytes per direction and GPU against 2 * n * (replicas - 1) / replicas
//    for peer accesses: the peer form moves less for two or three replicas, the multicast form
//    for four or more.
//
// 2. w2v_comm_* / w2v_allreduce_avg: the same average through NCCL, for hosts
//    that own the model buffers themselves (a JVM with one thread per GPU and
//    matrices allocated by its matrix library).  NCCL is loaded at run time
//    (libnccl.so.2), so the library has no link-time dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/bidmach_b200.h"
#include "w2v_internal.h"

namespace {

__device__ __forceinline__ float4 multimem_sum_v4(const float *mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ void multimem_store_v4(float *mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

constexpr int kAvgThreads = 512;
constexpr int kAvgUnroll = 4;

// mc: multicast address of the first float of this replica's slice; nvec 16-byte vectors.
__global__ void __launch_bounds__(kAvgThreads) nvls_average_kernel(float *mc, int64_t nvec, float scale) {
  const int64_t stride = (int64_t)gridDim.x * kAvgThreads;
  int64_t i = (int64_t)blockIdx.x * kAvgThreads + threadIdx.x;
  // four sums in flight per thread before the first store: the round trip through the switch
  // is long, and a CTA's throughput is what it keeps in flight over that latency
  for (; i + (kAvgUnroll - 1) * stride < nvec; i += kAvgUnroll * stride) {
    float4 v[kAvgUnroll];
#pragma unroll
    for (int u = 0; u < kAvgUnroll; u++) v[u] = multimem_sum_v4(mc + 4 * (i + u * stride));
#pragma unroll
    for (int u = 0; u < kAvgUnroll; u++) {
      v[u].x *= scale; v[u].y *= scale; v[u].z *= scale; v[u].w *= scale;
      multimem_store_v4(mc + 4 * (i + u * stride), v[u]);
    }
  }
  for (; i < nvec; i += stride) {
    float4 v = multimem_sum_v4(mc + 4 * i);
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    multimem_store_v4(mc + 4 * i, v);
  }
}

constexpr int kMaxPeers = 8;
struct PeerPtrs {
  float *p[kMaxPeers];
};

__device__ __forceinline__ float4 load_sys_v4(const float *a) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(a)
               : "memory");
  return v;
}

__device__ __forceinline__ void store_sys_v4(float *a, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// Every pointer addresses the same element of the buffer on one replica; first_vec / nvec
// delimit this replica's slice in 16-byte vectors.
template <int WORLD>
__global__ void __launch_bounds__(kAvgThreads) p2p_average_kernel(PeerPtrs pp, int64_t first_vec,
                                                                  int64_t nvec, float scale) {
  constexpr int U = WORLD <= 2 ? 4 : 2;   // vectors in flight per thread and replica
  const int64_t stride = (int64_t)gridDim.x * kAvgThreads;
  int64_t i = (int64_t)blockIdx.x * kAvgThreads + threadIdx.x;
  for (; i + (U - 1) * stride < nvec; i += U * stride) {
    float4 v[U][WORLD];
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
      for (int r = 0; r < WORLD; r++) v[u][r] = load_sys_v4(pp.p[r] + 4 * (first_vec + i + u * stride));
#pragma unroll
    for (int u = 0; u < U; u++) {
      float4 a = v[u][0];
#pragma unroll
      for (int r = 1; r < WORLD; r++) {
        a.x += v[u][r].x; a.y += v[u][r].y; a.z += v[u][r].z; a.w += v[u][r].w;
      }
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
#pragma unroll
      for (int r = 0; r < WORLD; r++) store_sys_v4(pp.p[r] + 4 * (first_vec + i + u * stride), a);
    }
  }
  for (; i < nvec; i += stride) {
    float4 a = load_sys_v4(pp.p[0] + 4 * (first_vec + i));
#pragma unroll
    for (int r = 1; r < WORLD; r++) {
      const float4 b = load_sys_v4(pp.p[r] + 4 * (first_vec + i));
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
#pragma unroll
    for (int r = 0; r < WORLD; r++) store_sys_v4(pp.p[r] + 4 * (first_vec + i), a);
  }
}

// ---- NCCL, bound at run time ------------------------------------------------
typedef void *nccl_comm_t;
struct nccl_unique_id { char internal[128]; };
enum { kNcclSuccess = 0, kNcclFloat = 7, kNcclSum = 0, kNcclAvg = 4 };  // public constants of nccl.h

struct NcclApi {
  void *handle = nullptr;
  int (*GetUniqueId)(nccl_unique_id *) = nullptr;
  int (*CommInitRank)(nccl_comm_t *, int, nccl_unique_id, int) = nullptr;
  int (*CommInitAll)(nccl_comm_t *, int, const int *) = nullptr;
  int (*CommDestroy)(nccl_comm_t) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*CommRegister)(nccl_comm_t, void *, size_t, void **) = nullptr;
  int (*CommDeregister)(nccl_comm_t, void *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
};

NcclApi *nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) return;
#define W2V_BIND(field, sym) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, sym))
    W2V_BIND(GetUniqueId, "ncclGetUniqueId");
    W2V_BIND(CommInitRank, "ncclCommInitRank");
    W2V_BIND(CommInitAll, "ncclCommInitAll");
    W2V_BIND(CommDestroy, "ncclCommDestroy");
    W2V_BIND(AllReduce, "ncclAllReduce");
    W2V_BIND(GroupStart, "ncclGroupStart");
    W2V_BIND(GroupEnd, "ncclGroupEnd");
    W2V_BIND(CommRegister, "ncclCommRegister");
    W2V_BIND(CommDeregister, "ncclCommDeregister");
    W2V_BIND(GetErrorString, "ncclGetErrorString");
#undef W2V_BIND
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommInitAll || !api.CommDestroy || !api.AllReduce ||
        !api.GroupStart || !api.GroupEnd)
      api.handle = nullptr;
  });
  return api.handle ? &api : nullptr;
}

// NCCL results are reported as 2000 + ncclResult_t, outside the range of cudaError_t values
int nccl_err(int r, const char *what) {
  if (r == kNcclSuccess) return 0;
  NcclApi *a = nccl();
  fprintf(stderr, "%s: NCCL error %d (%s)\n", what, r, (a && a->GetErrorString) ? a->GetErrorString(r) : "?");
  return 2000 + r;
}

}  // namespace

struct w2v_comm {
  nccl_comm_t comm;
  int nranks, rank, device;
  void *reg_buf;      // buffer registered with the communicator (zero-copy collectives), or null
  void *reg_handle;
};

extern "C" {

int w2v_nvls_average(float *mc_base, int64_t n, int rank, int world, int blocks, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!mc_base || world < 1 || rank < 0 || rank >= world || n < 0) return 1;
  if ((n & 3) || ((uintptr_t)mc_base & 15)) return 1;
  const int64_t nvec = n / 4;
  // slices in whole vectors; the last replica takes the remainder
  const int64_t per = nvec / world;
  const int64_t first = per * rank;
  const int64_t mine = (rank == world - 1) ? nvec - first : per;
  if (mine <= 0) return 0;
  if (blocks <= 0) blocks = w2v::device_sm_count();
  const int64_t need = (mine + kAvgThreads - 1) / kAvgThreads;
  if (blocks > need) blocks = (int)need;
  nvls_average_kernel<<<blocks, kAvgThreads, 0, stream>>>(mc_base + 4 * first, mine, 1.0f / (float)world);
  w2v::count_launch(1);
  return (int)cudaGetLastError();
}

int w2v_p2p_average(float *const *replicas_host, int64_t n, int rank, int world, int blocks, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!replicas_host || world < 1 || world > kMaxPeers || rank < 0 || rank >= world || n < 0) return 1;
  if (n & 3) return 1;
  PeerPtrs pp;
  for (int r = 0; r < kMaxPeers; r++) {
    // this replica's own copy first: its loads are the cheap ones and start the sums
    pp.p[r] = r < world ? replicas_host[(rank + r) % world] : nullptr;
    if (r < world && (!pp.p[r] || ((uintptr_t)pp.p[r] & 15))) return 1;
  }
  const int64_t nvec = n / 4;
  const int64_t per = nvec / world;
  const int64_t first = per * rank;
  const int64_t mine = (rank == world - 1) ? nvec - first : per;
  if (mine <= 0 || world == 1) return 0;
  if (blocks <= 0) blocks = w2v::device_sm_count();
  const int64_t need = (mine + kAvgThreads - 1) / kAvgThreads;
  if (blocks > need) blocks = (int)need;
  const float scale = 1.0f / (float)world;
  switch (world) {
    case 2: p2p_average_kernel<2><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
    case 3: p2p_average_kernel<3><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
    case 4: p2p_average_kernel<4><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
    case 5: p2p_average_kernel<5><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
    case 6: p2p_average_kernel<6><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
    case 7: p2p_average_kernel<7><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
    default: p2p_average_kernel<8><<<blocks, kAvgThreads, 0, stream>>>(pp, first, mine, scale); break;
  }
  w2v::count_launch(1);
  return (int)cudaGetLastError();
}

int w2v_comm_unique_id(void *id128) {
  if (!id128) return 1;
  NcclApi *a = nccl();
  if (!a) return 2;
  return nccl_err(a->GetUniqueId(reinterpret_cast<nccl_unique_id *>(id128)), "w2v_comm_unique_id");
}

int w2v_comm_init_rank(int nranks, int rank, const void *id128, w2v_comm **out) {
  if (!out || !id128 || nranks < 1 || rank < 0 || rank >= nranks) return 1;
  NcclApi *a = nccl();
  if (!a) return 2;
  w2v_comm *c = new w2v_comm();
  c->nranks = nranks;
  c->rank = rank;
  c->reg_buf = c->reg_handle = nullptr;
  cudaGetDevice(&c->device);
  int r = a->CommInitRank(&c->comm, nranks, *reinterpret_cast<const nccl_unique_id *>(id128), rank);
  if (r != kNcclSuccess) {
    delete c;
    return nccl_err(r, "w2v_comm_init_rank");
  }
  *out = c;
  return 0;
}

int w2v_comm_init_all(int ndev, const int *devices, w2v_comm **comms) {
  if (ndev < 1 || ndev > 64 || !comms) return 1;
  NcclApi *a = nccl();
  if (!a) return 2;
  nccl_comm_t raw[64];
  int r = a->CommInitAll(raw, ndev, devices);
  if (r != kNcclSuccess) return nccl_err(r, "w2v_comm_init_all");
  for (int i = 0; i < ndev; i++) {
    w2v_comm *c = new w2v_comm();
    c->comm = raw[i];
    c->nranks = ndev;
    c->rank = i;
    c->device = devices ? devices[i] : i;
    c->reg_buf = c->reg_handle = nullptr;
    comms[i] = c;
  }
  return 0;
}

int w2v_comm_register(w2v_comm *c, void *buf, int64_t bytes) {
  if (!c || !buf || bytes <= 0) return 1;
  NcclApi *a = nccl();
  if (!a) return 2;
  if (!a->CommRegister) return 0;   // an older NCCL: collectives work unregistered
  if (c->reg_handle && a->CommDeregister) a->CommDeregister(c->comm, c->reg_handle);
  c->reg_buf = c->reg_handle = nullptr;
  int r = a->CommRegister(c->comm, buf, (size_t)bytes, &c->reg_handle);
  if (r != kNcclSuccess) return nccl_err(r, "w2v_comm_register");
  c->reg_buf = buf;
  return 0;
}

int w2v_allreduce_avg(w2v_comm *c, float *A, float *B, int64_t n_each, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!c || n_each < 0 || (!A && !B)) return 1;
  if (n_each == 0 || c->nranks == 1) return 0;
  NcclApi *a = nccl();
  if (!a) return 2;
  if (A && B && B == A + n_each)   // both matrices in one buffer: one collective
    return nccl_err(a->AllReduce(A, A, (size_t)(2 * n_each), kNcclFloat, kNcclAvg, c->comm, stream),
                    "w2v_allreduce_avg");
  int r = a->GroupStart();
  if (r == kNcclSuccess && A) r = a->AllReduce(A, A, (size_t)n_each, kNcclFloat, kNcclAvg, c->comm, stream);
  if (r == kNcclSuccess && B) r = a->AllReduce(B, B, (size_t)n_each, kNcclFloat, kNcclAvg, c->comm, stream);
  int e = a->GroupEnd();
  return nccl_err(r != kNcclSuccess ? r : e, "w2v_allreduce_avg");
}

void w2v_comm_destroy(w2v_comm *c) {
  if (!c) return;
  NcclApi *a = nccl();
  if (a) {
    if (c->reg_handle && a->CommDeregister) a->CommDeregister(c->comm, c->reg_handle);
    a->CommDestroy(c->comm);
  }
  delete c;
}

}  // extern "C"
