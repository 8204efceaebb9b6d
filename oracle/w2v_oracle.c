/*
 * CPU oracle for the Word2Vec skip-gram negative-sampling minibatch path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, what the
 * reference computes on its CPU path so that the CUDA kernels can be checked
 * against it.  Nothing in the shipped library links, loads or calls it.
 *
 * Every function names the reference lines it follows (paths are relative to
 * the BIDMach source tree).  Arithmetic types are kept as the reference has
 * them: fp32 storage and fp32 accumulation, with the transcendental calls
 * (exp, pow, log) evaluated in double and rounded back, exactly where the
 * reference does so.  Row offsets are 64-bit here; the reference multiplies
 * `nrows * id` in a 32-bit int (jni/src/BIDMach_CPUMACH.c:31,40), which only
 * differs once dim*vocab exceeds 2^31 elements.
 *
 * Work is split into `nthreads` contiguous chunks of columns exactly as the
 * reference splits it (BIDMach_CPUMACH.c:23-24).  With nthreads == 1 the
 * result is deterministic; with more the chunks run concurrently under OpenMP
 * and race on shared rows without synchronisation, as the reference does.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static inline int chunk_lo(int t, int n, int nthreads) {
  return (int)(((int64_t)t * n) / nthreads);
}

/* Guarded logistic: BIDMach_CPUMACH.c:48-55 (same in :228-235, :400-407). */
static inline float guarded_sigmoid(float x) {
  if (x > 16.0f) return 1.0f;
  if (x < -16.0f) return 0.0f;
  float e = (float)exp((double)x);
  return e / (1.0f + e);
}

static inline float row_dot(const float *a, const float *b, int n) {
  float s = 0;
  for (int c = 0; c < n; c++) s += a[c] * b[c];
  return s;
}

/* (1 + id)^vexp evaluated in double, stored as float: BIDMach_CPUMACH.c:33,42. */
static inline float freq_scale(int id, float vexp) {
  return (float)pow((double)(1 + id), (double)vexp);
}

/*
 * Positive-pair update.  Follows Java_edu_berkeley_bid_CPUMACH_word2vecPos,
 * jni/src/BIDMach_CPUMACH.c:10-78 (Scala twin: networks/Word2Vec.scala:596-663).
 * A is indexed by the centre word, B by the context word.  The context row is
 * updated at once, the centre row after its whole window.
 */
ORC_API void orc_word2vecPos(int nrows, int ncols, int skip, const int *W, const int *LB,
                             const int *UB, float *A, float *B, float lrate, float vexp,
                             int nthreads) {
  (void)skip;
#pragma omp parallel for
  for (int t = 0; t < nthreads; t++) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)nrows);
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      int wc = W[i];
      if (wc < 0) continue;
      float *arow = A + (int64_t)nrows * wc;
      float sa = freq_scale(wc, vexp);
      memset(acc, 0, sizeof(float) * (size_t)nrows);
      for (int j = LB[i]; j <= UB[i]; j++) {
        if (j == 0 || i + j < 0 || i + j >= ncols) continue;
        int wx = W[i + j];
        if (wx < 0) continue;
        float *brow = B + (int64_t)nrows * wx;
        float sb = freq_scale(wx, vexp);
        float g = lrate * (1.0f - guarded_sigmoid(row_dot(arow, brow, nrows)));
        for (int c = 0; c < nrows; c++) {
          acc[c] += sa * g * brow[c];
          brow[c] += sb * g * arow[c];
        }
      }
      for (int c = 0; c < nrows; c++) arow[c] += acc[c];
    }
    free(acc);
  }
}

/*
 * Negative-pair update.  Follows Java_edu_berkeley_bid_CPUMACH_word2vecNeg,
 * jni/src/BIDMach_CPUMACH.c:186-264 (Scala twin: networks/Word2Vec.scala:760-849).
 * Column i pairs every one of its nwa A-words with every one of its nwb B-words.
 */
ORC_API void orc_word2vecNeg(int nrows, int ncols, int nwa, int nwb, const int *WA,
                             const int *WB, float *A, float *B, float lrate, float vexp,
                             int nthreads) {
#pragma omp parallel for
  for (int t = 0; t < nthreads; t++) {
    float *da = (float *)malloc(sizeof(float) * (size_t)nrows * nwa);
    float *db = (float *)malloc(sizeof(float) * (size_t)nrows);
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      const int *wa = WA + (int64_t)i * nwa;
      const int *wb = WB + (int64_t)i * nwb;
      memset(da, 0, sizeof(float) * (size_t)nrows * nwa);
      for (int k = 0; k < nwb; k++) {
        float *brow = B + (int64_t)nrows * wb[k];
        float sb = freq_scale(wb[k], vexp);
        memset(db, 0, sizeof(float) * (size_t)nrows);
        for (int j = 0; j < nwa; j++) {
          float *arow = A + (int64_t)nrows * wa[j];
          float sa = freq_scale(wa[j], vexp);
          float g = -lrate * guarded_sigmoid(row_dot(arow, brow, nrows));
          float *daj = da + (size_t)j * nrows;
          for (int c = 0; c < nrows; c++) {
            db[c] += sb * g * arow[c];
            daj[c] += sa * g * brow[c];
          }
        }
        for (int c = 0; c < nrows; c++) brow[c] += db[c];
      }
      for (int j = 0; j < nwa; j++) {
        float *arow = A + (int64_t)nrows * wa[j];
        const float *daj = da + (size_t)j * nrows;
        for (int c = 0; c < nrows; c++) arow[c] += daj[c];
      }
    }
    free(db);
    free(da);
  }
}

/*
 * Sum of log sigma(a.b) over the positive pairs.  Follows Word2Vec.evalPosCPU,
 * networks/Word2Vec.scala:953-1005: fp32 dot and sigmoid, then
 * log(max((double)s, 1e-20)) summed in double.  (The C twin,
 * BIDMach_CPUMACH.c:368-427, clamps at 1e-40 and returns an uninitialised
 * accumulator, so the Scala version is the one restated.)
 */
ORC_API double orc_word2vecEvalPos(int nrows, int ncols, int skip, const int *W, const int *LB,
                                   const int *UB, const float *A, const float *B, int nthreads) {
  (void)skip;
  double total = 0;
#pragma omp parallel for reduction(+ : total)
  for (int t = 0; t < nthreads; t++) {
    double part = 0;
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      int wc = W[i];
      if (wc < 0) continue;
      const float *arow = A + (int64_t)nrows * wc;
      for (int j = LB[i]; j <= UB[i]; j++) {
        if (j == 0 || i + j < 0 || i + j >= ncols) continue;
        int wx = W[i + j];
        if (wx < 0) continue;
        float s = guarded_sigmoid(row_dot(arow, B + (int64_t)nrows * wx, nrows));
        part += log(fmax((double)s, 1e-20));
      }
    }
    total += part;
  }
  return total;
}

/*
 * Sum of log(1 - sigma(a.b)) over all nwa*nwb pairs of every column.  Follows
 * Word2Vec.evalNegCPU, networks/Word2Vec.scala:1071-1132 (1 - s is formed in
 * fp32 there, then widened).
 */
ORC_API double orc_word2vecEvalNeg(int nrows, int ncols, int nwa, int nwb, const int *WA,
                                   const int *WB, const float *A, const float *B, int nthreads) {
  double total = 0;
#pragma omp parallel for reduction(+ : total)
  for (int t = 0; t < nthreads; t++) {
    double part = 0;
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      for (int k = 0; k < nwb; k++) {
        const float *brow = B + (int64_t)nrows * WB[(int64_t)i * nwb + k];
        for (int j = 0; j < nwa; j++) {
          const float *arow = A + (int64_t)nrows * WA[(int64_t)i * nwa + j];
          float s = guarded_sigmoid(row_dot(arow, brow, nrows));
          part += log(fmax((double)(1.0f - s), 1e-20));
        }
      }
    }
    total += part;
  }
  return total;
}

/*
 * Vocabulary slices.  mapIndx (BIDMach_CPUMACH.c:80-88; networks/Word2Vec.scala:665-672) with the
 * model of a slice held as one matrix per side (the reference cuts it into blocks of maxCols words
 * because a Java array is limited to 2^31 elements): ids below nhead have a row on every slice,
 * an id at or above it belongs to slice id % nslices and sits at row (id - nhead) / nslices + nhead.
 */
typedef struct {
  int64_t row;
  int mine, head;
} orc_slot;

static inline orc_slot slice_slot(int id, int islice, int nslices, int nhead) {
  orc_slot s;
  s.row = (id >= nhead) ? (id - nhead) / nslices + nhead : id;
  s.mine = (id >= nhead) && (id % nslices == islice);
  s.head = (id < nhead);
  return s;
}

static inline int slice_pair(orc_slot a, orc_slot b, int do_head) {
  return (do_head > 1 && a.head && b.head) || (a.mine && b.head) || (b.mine && a.head) ||
         (a.mine && b.mine);
}

/* Follows Java_edu_berkeley_bid_CPUMACH_word2vecPosSlice, BIDMach_CPUMACH.c:90-184. */
ORC_API void orc_word2vecPosSlice(int nrows, int ncols, int skip, const int *W, const int *LB,
                                  const int *UB, float *A, float *B, float lrate, float vexp,
                                  int nthreads, int islice, int nslices, int nhead, int do_head) {
  (void)skip;
#pragma omp parallel for
  for (int t = 0; t < nthreads; t++) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)nrows);
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      int wc = W[i];
      if (wc < 0) continue;
      orc_slot sa_ = slice_slot(wc, islice, nslices, nhead);
      float *arow = A + (int64_t)nrows * sa_.row;
      float sa = freq_scale(wc, vexp);
      int touched = 0;
      memset(acc, 0, sizeof(float) * (size_t)nrows);
      for (int j = LB[i]; j <= UB[i]; j++) {
        if (j == 0 || i + j < 0 || i + j >= ncols) continue;
        int wx = W[i + j];
        if (wx < 0) continue;
        orc_slot sb_ = slice_slot(wx, islice, nslices, nhead);
        if (!slice_pair(sa_, sb_, do_head)) continue;
        float *brow = B + (int64_t)nrows * sb_.row;
        float sb = freq_scale(wx, vexp);
        touched = 1;
        float g = lrate * (1.0f - guarded_sigmoid(row_dot(arow, brow, nrows)));
        for (int c = 0; c < nrows; c++) acc[c] += sa * g * brow[c];
        if (sb_.mine || (sb_.head && do_head))
          for (int c = 0; c < nrows; c++) brow[c] += sb * g * arow[c];
      }
      if (touched && (sa_.mine || (sa_.head && do_head)))
        for (int c = 0; c < nrows; c++) arow[c] += acc[c];
    }
    free(acc);
  }
}

/* Follows Java_edu_berkeley_bid_CPUMACH_word2vecNegSlice, BIDMach_CPUMACH.c:267-366. */
ORC_API void orc_word2vecNegSlice(int nrows, int ncols, int nwa, int nwb, const int *WA,
                                  const int *WB, float *A, float *B, float lrate, float vexp,
                                  int nthreads, int islice, int nslices, int nhead, int do_head) {
#pragma omp parallel for
  for (int t = 0; t < nthreads; t++) {
    float *da = (float *)malloc(sizeof(float) * (size_t)nrows * nwa);
    float *db = (float *)malloc(sizeof(float) * (size_t)nrows);
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      const int *wa = WA + (int64_t)i * nwa;
      const int *wb = WB + (int64_t)i * nwb;
      memset(da, 0, sizeof(float) * (size_t)nrows * nwa);
      for (int k = 0; k < nwb; k++) {
        orc_slot sb_ = slice_slot(wb[k], islice, nslices, nhead);
        float *brow = B + (int64_t)nrows * sb_.row;
        float sb = freq_scale(wb[k], vexp);
        memset(db, 0, sizeof(float) * (size_t)nrows);
        for (int j = 0; j < nwa; j++) {
          orc_slot sa_ = slice_slot(wa[j], islice, nslices, nhead);
          if (!slice_pair(sa_, sb_, do_head)) continue;
          float *arow = A + (int64_t)nrows * sa_.row;
          float sa = freq_scale(wa[j], vexp);
          float g = -lrate * guarded_sigmoid(row_dot(arow, brow, nrows));
          float *daj = da + (size_t)j * nrows;
          for (int c = 0; c < nrows; c++) {
            db[c] += sb * g * arow[c];
            daj[c] += sa * g * brow[c];
          }
        }
        if (sb_.mine || (sb_.head && do_head))
          for (int c = 0; c < nrows; c++) brow[c] += db[c];
      }
      for (int j = 0; j < nwa; j++) {
        orc_slot sa_ = slice_slot(wa[j], islice, nslices, nhead);
        if (!(sa_.mine || (sa_.head && do_head))) continue;
        float *arow = A + (int64_t)nrows * sa_.row;
        const float *daj = da + (size_t)j * nrows;
        for (int c = 0; c < nrows; c++) arow[c] += daj[c];
      }
    }
    free(db);
    free(da);
  }
}

/* Follows Word2Vec.evalPosCPUslice, networks/Word2Vec.scala:1007-1068: the pairs whose two
 * words both have a row on this slice (head or mine), head-head pairs included. */
ORC_API double orc_word2vecEvalPosSlice(int nrows, int ncols, int skip, const int *W, const int *LB,
                                        const int *UB, const float *A, const float *B, int nthreads,
                                        int islice, int nslices, int nhead) {
  (void)skip;
  double total = 0;
#pragma omp parallel for reduction(+ : total)
  for (int t = 0; t < nthreads; t++) {
    double part = 0;
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      int wc = W[i];
      if (wc < 0) continue;
      orc_slot sa_ = slice_slot(wc, islice, nslices, nhead);
      if (!(sa_.mine || sa_.head)) continue;
      const float *arow = A + (int64_t)nrows * sa_.row;
      for (int j = LB[i]; j <= UB[i]; j++) {
        if (j == 0 || i + j < 0 || i + j >= ncols) continue;
        int wx = W[i + j];
        if (wx < 0) continue;
        orc_slot sb_ = slice_slot(wx, islice, nslices, nhead);
        if (!(sb_.mine || sb_.head)) continue;
        float s = guarded_sigmoid(row_dot(arow, B + (int64_t)nrows * sb_.row, nrows));
        part += log(fmax((double)s, 1e-20));
      }
    }
    total += part;
  }
  return total;
}

/* Follows Word2Vec.evalNegCPUslice, networks/Word2Vec.scala:1134-1200. */
ORC_API double orc_word2vecEvalNegSlice(int nrows, int ncols, int nwa, int nwb, const int *WA,
                                        const int *WB, const float *A, const float *B, int nthreads,
                                        int islice, int nslices, int nhead) {
  double total = 0;
#pragma omp parallel for reduction(+ : total)
  for (int t = 0; t < nthreads; t++) {
    double part = 0;
    int hi = chunk_lo(t + 1, ncols, nthreads);
    for (int i = chunk_lo(t, ncols, nthreads); i < hi; i++) {
      for (int k = 0; k < nwb; k++) {
        orc_slot sb_ = slice_slot(WB[(int64_t)i * nwb + k], islice, nslices, nhead);
        if (!(sb_.mine || sb_.head)) continue;
        const float *brow = B + (int64_t)nrows * sb_.row;
        for (int j = 0; j < nwa; j++) {
          orc_slot sa_ = slice_slot(WA[(int64_t)i * nwa + j], islice, nslices, nhead);
          if (!(sa_.mine || sa_.head)) continue;
          float s = guarded_sigmoid(row_dot(A + (int64_t)nrows * sa_.row, brow, nrows));
          part += log(fmax((double)(1.0f - s), 1e-20));
        }
      }
    }
    total += part;
  }
  return total;
}

/*
 * Frequent-word subsampling and window bounds.  Follows Word2Vec.wordMats,
 * networks/Word2Vec.scala:214-241, element by element:
 *   - the minibatch is a 2 x ncols int32 matrix stored column-major; row 0 is
 *     the word id and row 1 the sentence id (swapped when iflip)        :216-217,233
 *   - keep a word iff id < vocab and u1 < sqrt(x) + x with
 *     x = float(id + 1) * salpha, all in fp32                           :218-225
 *   - ubrand = min(nskip, int(u2 * nskip) + 1), lbrand = -ubrand        :228-230
 *   - lbsentence = 1 - (1-based position inside the run of equal
 *     sentence ids), ubsentence = (positions left in the run) - 1       :233-235
 *   - lb = max(lbrand, lbsentence), ub = min(ubrand, ubsentence)        :236-237
 * salpha = wsample * ln(vocab) in fp32 is formed by the caller (:150).
 */
ORC_API void orc_wordmats_bounds(int ncols, const int *wordsens, int iflip, int vocab, int nskip,
                                 float salpha, const float *u1, const float *u2, int *words,
                                 int *lb, int *ub) {
  int wrow = iflip ? 1 : 0;
  int srow = 1 - wrow;
  for (int i = 0; i < ncols; i++) {
    int id = wordsens[2 * i + wrow];
    int good = id < vocab;
    float x = (float)(id + 1) * salpha;
    float thr = sqrtf(x) + x;
    good = good && (u1[i] < thr);
    words[i] = good * (id + 1) - 1;
  }
  int run = 0;
  for (int i = 0; i < ncols; i++) {
    if (i == 0 || wordsens[2 * i + srow] != wordsens[2 * (i - 1) + srow]) run = 0;
    run += 1;
    int ubr = (int)(u2[i] * (float)nskip) + 1;
    if (ubr > nskip) ubr = nskip;
    int lbs = 1 - run;
    lb[i] = (-ubr > lbs) ? -ubr : lbs;
    ub[i] = ubr;
  }
  run = 0;
  for (int i = ncols - 1; i >= 0; i--) {
    if (i == ncols - 1 || wordsens[2 * i + srow] != wordsens[2 * (i + 1) + srow]) run = 0;
    run += 1;
    int ubs = run - 1;
    if (ubs < ub[i]) ub[i] = ubs;
  }
}

/*
 * Number of (centre, context) pairs the minibatch yields.  Follows the counting
 * loop of Word2Vec.getnegs, networks/Word2Vec.scala:283-302.
 */
ORC_API int64_t orc_count_pairs(int ncols, const int *words, const int *lb, const int *ub) {
  int64_t n = 0;
  for (int i = 0; i < ncols; i++) {
    if (words[i] < 0) continue;
    for (int j = lb[i]; j <= ub[i]; j++)
      if (j != 0 && words[i + j] >= 0) n++;
  }
  return n;
}

/*
 * Ordered list of good context words: centre ascending, offset ascending.
 * Follows the fill loop of Word2Vec.getnegs, networks/Word2Vec.scala:309-330,
 * for one thread (the reference's per-thread start offsets `ccc(ithread) -
 * ccc(0)` at :314 are only right for nthreads == 1, which is the case this
 * oracle pins).  Writes at most `cap` entries; returns how many it wrote.
 */
ORC_API int64_t orc_fill_contexts(int ncols, const int *words, const int *lb, const int *ub,
                                  int *ctx, int64_t cap) {
  int64_t n = 0;
  for (int i = 0; i < ncols; i++) {
    if (words[i] < 0) continue;
    for (int j = lb[i]; j <= ub[i] && n < cap; j++)
      if (j != 0 && words[i + j] >= 0) ctx[n++] = words[i + j];
  }
  return n;
}

/*
 * In-place random permutation with caller-supplied doubles in [0,1).  Follows
 * the serial shuffle of Word2Vec.getnegs, networks/Word2Vec.scala:336-346.
 */
ORC_API void orc_shuffle(int64_t n, int *ctx, const double *prand) {
  for (int64_t i = 0; i < n; i++) {
    int64_t pick = i + (int64_t)floor(prand[i] * (double)(n - i));
    if (pick > n - 1) pick = n - 1;
    if (pick > i) {
      int tmp = ctx[i];
      ctx[i] = ctx[pick];
      ctx[pick] = tmp;
    }
  }
}

/*
 * Negative word ids from uniforms: min(vocab-1, (int)(vocab * u^expt)) with the
 * power taken in double.  Follows Word2Vec.getnegs, networks/Word2Vec.scala:356
 * (expt = 1/(1 - wexpt) is formed in fp32 by the caller, :139).
 */
ORC_API void orc_negative_ids(int64_t n, const float *u, float expt, int vocab, int *out) {
  for (int64_t i = 0; i < n; i++) {
    double v = (double)vocab * pow((double)u[i], (double)expt);
    int id = (v >= 2147483647.0) ? 2147483647 : (int)v;
    out[i] = id < vocab - 1 ? id : vocab - 1;
  }
}

/* Size of the OpenMP team the chunked loops above really get: launchers such as
 * torch.distributed.run export OMP_NUM_THREADS=1, under which `nthreads` chunks run one
 * after the other.  n > 0 sets the team size first. */
ORC_API int orc_set_threads(int n) {
  int got = 0;
  if (n > 0) omp_set_num_threads(n);
#pragma omp parallel
  {
#pragma omp single
    got = omp_get_num_threads();
  }
  return got;
}
