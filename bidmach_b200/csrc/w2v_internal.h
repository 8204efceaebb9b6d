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
int thread_hot_rows(HotRows *out);

int eval_scratch(EvalScratch **out);
int take_stage_fault();  // nonzero (cudaErrorLaunchTimeout) if a staged kernel gave up waiting
int device_sm_count();
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
int pos_eval_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W, const int *LB,
                   const int *UB, const float *A, const float *B, float *retval,
                   cudaStream_t stream);
int neg_update_async(int dim, int ncols, const int *ncols_dev, int nwords, int nwa, int nwb,
                     const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                     const HotRows &hot, cudaStream_t stream);
int neg_eval_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                   const int *WB, const float *A, const float *B, float *retval,
                   cudaStream_t stream);
// Memory side only of the negative kernels on the same columns: mode 0 adds zeros to
// every row with the update kernel's reductions, mode 1 reads every row.
int row_probe_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                    const int *WB, float *A, float *B, const HotRows &hot, int mode, float *sink,
                    cudaStream_t stream);

}  // namespace w2v
