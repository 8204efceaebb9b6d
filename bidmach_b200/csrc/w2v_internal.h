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

int eval_scratch(EvalScratch **out);
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
                     cudaStream_t stream);
int pos_eval_async(int dim, int ncols, const int *ncols_dev, int skip, const int *W, const int *LB,
                   const int *UB, const float *A, const float *B, float *retval,
                   cudaStream_t stream);
int neg_update_async(int dim, int ncols, const int *ncols_dev, int nwords, int nwa, int nwb,
                     const int *WA, const int *WB, float *A, float *B, float lrate, float vexp,
                     cudaStream_t stream);
int neg_eval_async(int dim, int ncols, const int *ncols_dev, int nwa, int nwb, const int *WA,
                   const int *WB, const float *A, const float *B, float *retval,
                   cudaStream_t stream);

}  // namespace w2v
