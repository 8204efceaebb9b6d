// A consumer of the C ABI that has nothing to do with Python or PyTorch: it
// includes include/bidmach_b200.h, links libbidmachcuda-linux-x86_64.so, owns
// its device buffers through the CUDA runtime and calls the reference-named
// entry points the way BIDMach's JNI layer does.
//
//   cabi_consumer <input file> <output file>
//
// input  : int32 dim, vocab, ncols, nwa, nwb; float32 lrate, vexp;
//          int32 WA[ncols*nwa], WB[ncols*nwb]; float32 A[vocab*dim], B[vocab*dim]
// output : float32 score_before, score_before_noalloc, A[vocab*dim], B[vocab*dim] after word2vecNeg
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "bidmach_b200.h"

#define CK(x)                                                                   \
  do {                                                                          \
    cudaError_t e_ = (x);                                                       \
    if (e_ != cudaSuccess) {                                                    \
      fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));           \
      return 2;                                                                 \
    }                                                                           \
  } while (0)

int main(int argc, char **argv) {
  if (argc != 3) return 64;
  FILE *f = fopen(argv[1], "rb");
  if (!f) return 65;
  int hdr[5];
  float sc[2];
  if (fread(hdr, 4, 5, f) != 5 || fread(sc, 4, 2, f) != 2) return 66;
  const int dim = hdr[0], vocab = hdr[1], ncols = hdr[2], nwa = hdr[3], nwb = hdr[4];
  std::vector<int> WA((size_t)ncols * nwa), WB((size_t)ncols * nwb);
  std::vector<float> A((size_t)vocab * dim), B((size_t)vocab * dim);
  if (fread(WA.data(), 4, WA.size(), f) != WA.size() || fread(WB.data(), 4, WB.size(), f) != WB.size() ||
      fread(A.data(), 4, A.size(), f) != A.size() || fread(B.data(), 4, B.size(), f) != B.size())
    return 67;
  fclose(f);

  int *dWA, *dWB;
  float *dA, *dB, *dRet;
  CK(cudaMalloc(&dWA, WA.size() * 4));
  CK(cudaMalloc(&dWB, WB.size() * 4));
  CK(cudaMalloc(&dA, A.size() * 4));
  CK(cudaMalloc(&dB, B.size() * 4));
  CK(cudaMalloc(&dRet, 8));
  CK(cudaMemcpy(dWA, WA.data(), WA.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dWB, WB.data(), WB.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dA, A.data(), A.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dB, B.data(), B.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemset(dRet, 0, 8));

  int err = word2vecEvalNeg(dim, ncols, nwa, nwb, dWA, dWB, dA, dB, dRet);
  if (err) { fprintf(stderr, "word2vecEvalNeg: %s\n", cudaGetErrorString((cudaError_t)err)); return 3; }
  err = word2vecEvalNegNoAlloc(dim, ncols, nwa, nwb, dWA, dWB, dA, dB, dRet + 1);
  if (err) { fprintf(stderr, "word2vecEvalNegNoAlloc: %s\n", cudaGetErrorString((cudaError_t)err)); return 4; }
  err = word2vecNeg(dim, ncols, nwa, nwb, dWA, dWB, dA, dB, sc[0], sc[1]);
  if (err) { fprintf(stderr, "word2vecNeg: %s\n", cudaGetErrorString((cudaError_t)err)); return 5; }
  // the reference's error convention: an unsupported shape returns 1 and touches nothing
  if (word2vecNeg(dim, ncols, 3, 3, dWA, dWB, dA, dB, sc[0], sc[1]) != 1) return 6;

  float scores[2];
  CK(cudaMemcpy(scores, dRet, 8, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(A.data(), dA, A.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(B.data(), dB, B.size() * 4, cudaMemcpyDeviceToHost));
  FILE *g = fopen(argv[2], "wb");
  if (!g) return 68;
  fwrite(scores, 4, 2, g);
  fwrite(A.data(), 4, A.size(), g);
  fwrite(B.data(), 4, B.size(), g);
  fclose(g);

  // the whole-minibatch calls from plain C++: a context, a model, a pinned host minibatch
  // trained on eight times and scored before and after
  {
    w2v_opts o;
    w2v_default_opts(&o);
    o.dim = 100;
    o.vocabSize = 500;
    o.wsample = 1.0f;
    o.lrate = 0.01f;
    o.seed = 5;
    const int n = 3000;
    w2v_ctx *ctx = nullptr;
    if (w2v_create(&o, n, &ctx) != 0) return 7;
    float *mA, *mB;
    CK(cudaMalloc(&mA, sizeof(float) * o.dim * o.vocabSize));
    CK(cudaMalloc(&mB, sizeof(float) * o.dim * o.vocabSize));
    if (w2v_init_model(&o, mA, mB, nullptr) != 0) return 8;
    int *toks;
    CK(cudaMallocHost(&toks, sizeof(int) * 2 * n));
    unsigned x = 12345u;
    for (int i = 0; i < n; i++) {
      x = x * 1664525u + 1013904223u;
      toks[2 * i] = (int)((x >> 8) % (unsigned)o.vocabSize);
      toks[2 * i + 1] = i / 37;
    }
    double before = 0, after = 0;
    if (w2v_evalbatch_host(ctx, toks, mA, mB, 1, &before, nullptr) != 0) return 9;
    long long pairs = 0;
    for (int k = 0; k < 8; k++) {
      int64_t np = 0;
      if (w2v_dobatch_host(ctx, toks, mA, mB, n, 2 + k, &np, nullptr) != 0) return 10;
      pairs = np;
    }
    if (w2v_evalbatch_host(ctx, toks, mA, mB, 20, &after, nullptr) != 0) return 11;
    printf("minibatch pairs=%lld score %.6f -> %.6f\n", pairs, before, after);
    w2v_destroy(ctx);
    CK(cudaFreeHost(toks));
    CK(cudaFree(mA));
    CK(cudaFree(mB));
  }
  printf("ok launches=%lld\n", w2v_launch_count());
  return 0;
}
