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
// Vocabulary slicing of the reference's multi-node mode (Word2Vec.Opts nSlices / iSlice /
// nHeadTerms / doHead; mapIndx, networks/Word2Vec.scala:665-672 and BIDMach_CPUMACH.c:80-88):
// ids below `nhead` (the head) have a row on every slice, an id at or above it belongs to slice
// `id % nslices` and is stored there at row (id - nhead) / nslices + nhead.  A pair is worked on
// when both of its words have a row here, except head-head pairs unless do_head > 1; head rows
// are written only when do_head > 0.  nslices == 1 with nhead == 0 is the whole vocabulary.
struct SliceMap {
  int nhead, nslices, islice, do_head;
  __host__ __device__ bool whole() const { return nslices <= 1; }
  // row of a global id on this slice, or -1 when the slice holds none
  __host__ __device__ int local(int id) const {
    if (id < nhead) return id;   // head ids, and a masked id (-1) as it is
    if (id % nslices != islice) return -1;
    return (id - nhead) / nslices + nhead;
  }
  // the global id stored at a local row (what the per-word rate scale is computed from)
  __host__ __device__ int global(int row) const {
    if (row < nhead) return row;
    int r = (islice - nhead) % nslices;
    if (r < 0) r += nslices;
    return nhead + (row - nhead) * nslices + r;
  }
  __host__ __device__ bool skips_head_pairs() const { return do_head <= 1; }
  __host__ __device__ bool freezes_head() const { return do_head <= 0; }
};
inline SliceMap whole_vocabulary() { return SliceMap{0, 1, 0, 1}; }

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
// `slice` other than whole_vocabulary(): W / WA / WB hold global ids, A and B the rows of this
// slice only (see SliceMap).
int pos_update_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W,
                     const int *LB, const int *UB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, const SliceMap &slice, cudaStream_t stream);
// `scratch` is the caller's zeroed accumulator (the kernels leave it zeroed again); `fault`
// is where a staged kernel that gave up waiting for its copies writes 1 (host-visible memory).
int pos_eval_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W, const int *LB,
                   const int *UB, const float *A, const float *B, float *retval,
                   EvalScratch *scratch, const SliceMap &slice, cudaStream_t stream);
int neg_update_async(int dim, int ncols, const int *ncols_dev, int nwords, int nwa, int nwb,
                     const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, int *fault, const SliceMap &slice, cudaStream_t stream);
int neg_eval_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                   const int *WB, const float *A, const float *B, float *retval,
                   EvalScratch *scratch, int *fault, const SliceMap &slice, cudaStream_t stream);

}  // namespace w2v
