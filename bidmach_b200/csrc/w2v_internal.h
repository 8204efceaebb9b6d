// Internal interfaces between the translation units of libbidmachcuda.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace w2v {

// Double-precision accumulator the eval kernels share across blocks; the last
// block to arrive moves the total out and re-arms it.
struct EvalScratch {
  double sum;
  unsigned arrived;
  unsigned pad;
};

// Side buffer of replica rows for the most frequent word ids (see
// w2v_kernels.cu).  limit = 2^levels: ids with id + 1 < limit are hot; 0 = off.
struct HotRows {
  float *shadowA;
  float *shadowB;
  int limit;
  int rmax;        // replicas of id 0 (a power of two); level L ids have rmax >> L
  int fold_every;  // in-kernel folding period (0 = only the fold kernel folds)
  // Optional: {kept tokens, kept tokens of word 0} of the minibatch, on the device.  With
  // them the kernels shorten the folding period when the text is dense and the rate high
  // (see fold_period in w2v_kernels.cu); null = fold_every as it stands.
  const int *stats;
};
size_t hot_rows_bytes();
int hot_levels_default();
HotRows hot_rows_at(float *zeroed_buffer, int levels);

// Scratch memory of one synchronous launcher call (word2vecPos ... word2vecEvalNeg): replica
// rows, the hot-word counts of the launch, the scoring accumulator, and a flag in pinned host
// memory that a staged kernel raises when it gave up waiting for its copies.  Sets are kept
// in one pool per device and handed out for the duration of a call, so their number follows
// the number of calls in flight on that device, not the number of host threads that ever
// called (a host that starts fresh threads for every training run leaks nothing).
struct LaunchScratch {
  float *hot_buf;    // replica rows, all zero between calls
  int *stats;        // device int[2]: {valid ids, ids equal to 0} of the launch's word list
  EvalScratch *eval; // zero between calls
  int *fault;        // pinned host int, also addressable from the device
  int device;
  LaunchScratch *next;
};
int acquire_launch_scratch(LaunchScratch **out);   // 0 or a cudaError_t
void release_launch_scratch(LaunchScratch *s);

// Counts the ids in [0, nwords) and the ids equal to 0 among ids[0..n) into stats[0..1]
// (cleared first), on `stream`: the hot-word share that fold_period needs, for callers
// that did not run the library's own preprocessing.
int count_hot_share_async(const int *ids, int64_t n, int nwords, int *stats, cudaStream_t stream);

// SMs of the current device that the calling thread's launches may fill: all of them, less
// what an SmReserve in scope on this thread holds back for a kernel on another stream.
int device_sm_count();
struct SmReserve {
  explicit SmReserve(int sms);
  ~SmReserve();
  int previous;
};
long long launch_count();
void count_launch(int n);
bool neg_shape_supported(int nwa, int nwb);

// Launch-only forms of the four kernels.  `ncols_dev`, when not null, is a
// device int that overrides `ncols` inside the kernel (so a column count
// produced on the device never has to visit the host); `ncols` is then only an
// upper bound used to size the grid.
int pos_update_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W,
                     const int *LB, const int *UB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, cudaStream_t stream);
// `scratch` is the caller's zeroed accumulator (the kernels leave it zeroed again); `fault`
// is where a staged kernel that gave up waiting for its copies writes 1 (host-visible memory).
int pos_eval_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W, const int *LB,
                   const int *UB, const float *A, const float *B, float *retval,
                   EvalScratch *scratch, cudaStream_t stream);
int neg_update_async(int dim, int ncols, const int *ncols_dev, int nwords, int nwa, int nwb,
                     const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, int *fault, cudaStream_t stream);
int neg_eval_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                   const int *WB, const float *A, const float *B, float *retval,
                   EvalScratch *scratch, int *fault, cudaStream_t stream);

}  // namespace w2v
