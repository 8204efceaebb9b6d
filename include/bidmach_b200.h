/*
 * libbidmachcuda-linux-x86_64.so -- C ABI of the B200 (sm_100a) Word2Vec
 * skip-gram negative-sampling path.
 *
 * Part 1 and part 2 are the drop-in surface: exactly the functions that the
 * JVM side of BIDMach binds for this path (edu.berkeley.bid.CUMACH) and the C
 * launchers underneath them.  Part 3 is an extension for callers that want the
 * whole minibatch (preprocessing + update, or preprocessing + scoring) in one
 * call.  No function takes or returns anything but plain pointers and scalars.
 *
 * Conventions common to all of it
 *   - model matrices are column-major dim x vocab fp32 in device memory: word w
 *     is the contiguous row [w*dim, (w+1)*dim).  `A` is the matrix indexed by
 *     centre and negative words (modelmats(1) in BIDMach), `B` the one indexed
 *     by context words (modelmats(0), the exported embedding).
 *   - every pointer is a device pointer unless its name ends in `_host`.
 *   - buffers are owned by the caller; the library never frees or keeps them.
 *   - return value: 0 on success, otherwise a cudaError_t value (feed it to
 *     cudaGetErrorString), or 1 for an unsupported shape, as the reference does.
 *   - the library uses the CUDA device that is current on the calling thread.
 */
#ifndef BIDMACH_B200_H
#define BIDMACH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------
 * Part 1 -- launchers with the reference's prototypes.
 * Each runs on the calling thread's default stream and returns after the
 * kernel has finished (the reference synchronises the same way,
 * jni/src/DNN127.cu:1417-1419).
 * ---------------------------------------------------------------------- */

/* Replaces word2vecPos, jni/include/MatKernel.hpp:77 (launcher
 * jni/src/DNN127.cu:1389-1420).  W/LB/UB are int32[ncols].  `shift` is the
 * window half-width and must be 2, 3 or 5; nrows (= dim) must be <= 1280;
 * otherwise a line is printed and 1 is returned. */
int word2vecPos(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                float lrate, float vexp);

/* Replaces word2vecNeg, jni/include/MatKernel.hpp:79 (launcher
 * jni/src/DNN127.cu:1423-1452).  WA is int32[nwa x ncols], WB int32[nwb x ncols],
 * both column-major (column c contiguous).  (nwa, nwb) must be one of (5,1),
 * (5,5), (10,5), (5,10); otherwise a line is printed and 1 is returned. */
int word2vecNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                float lrate, float vexp);

/* Replaces word2vecNegFilt, jni/include/MatKernel.hpp:81 (launcher
 * jni/src/DNN127.cu:1454-1483): as word2vecNeg, but a word id >= nwords acts
 * as a zero row and is not updated. */
int word2vecNegFilt(int nrows, int ncols, int nwords, int nwa, int nwb, int *WA, int *WB, float *A,
                    float *B, float lrate, float vexp);

/* Replaces word2vecEvalPos, jni/include/MatKernel.hpp:83 (launcher
 * jni/src/DNN127.cu:1485-1516).  Adds the sum of log(max(sigmoid(a.b),1e-20))
 * over the positive pairs to the device float Retval[0]; the caller clears it
 * first (networks/Word2Vec.scala:476). */
int word2vecEvalPos(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                    float *Retval);

/* Replaces word2vecEvalNeg, jni/include/MatKernel.hpp:85 (launcher
 * jni/src/DNN127.cu:1519-1548).  Adds the sum of log(max(1-sigmoid(a.b),1e-20))
 * over all nwa*nwb pairs of every column to Retval[0]. */
int word2vecEvalNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                    float *Retval);

/* No counterpart in the reference.  Same contract as word2vecEvalNeg, for
 * hosts that must not allocate device memory while they run (a JVM whose matrix
 * cache already owns the card, a process that froze its memory map, work being
 * recorded into a stream capture): the partial sums live in an array built into
 * the library's device image (about 64 KiB on every GPU that loads the library)
 * instead of a buffer obtained with cudaMalloc.  At most 2,097,152 columns per
 * call; a larger ncols prints a message and returns 1.  The first call on a
 * device looks up the array's device address and should therefore be made
 * outside any stream capture.  Calls on the same GPU share the array: do not
 * let two of them run at the same time. */
int word2vecEvalNegNoAlloc(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A,
                           float *B, float *Retval);

/* ------------------------------------------------------------------------
 * Part 2 -- JNI entry points, bound by name from edu.berkeley.bid.CUMACH
 * (src/main/java/edu/berkeley/bid/CUMACH.java:90-98).  They replace the
 * functions of the same name in jni/src/BIDMach_CUMACH.cpp:434-493 and
 * JNI_OnLoad at :11-29.  JNIEnv / jobject are opaque here; every jobject
 * argument is a jcuda.Pointer whose device address is nativePointer +
 * byteOffset (jni/src/PointerUtils.cpp:353-363); a null object is a null
 * pointer.
 * ---------------------------------------------------------------------- */
#ifndef BIDMACH_B200_NO_JNI_DECLS
struct BidmachJNIEnv_;
typedef const struct BidmachJNIEnv_ *BidmachJNIEnv;

int JNI_OnLoad(void *jvm, void *reserved);
int Java_edu_berkeley_bid_CUMACH_word2vecPos(BidmachJNIEnv *env, void *obj, int nrows, int ncols,
                                             int shift, void *jW, void *jLB, void *jUB, void *jA,
                                             void *jB, float lrate, float vexp);
int Java_edu_berkeley_bid_CUMACH_word2vecNeg(BidmachJNIEnv *env, void *obj, int nrows, int ncols,
                                             int nwa, int nwb, void *jWA, void *jWB, void *jA,
                                             void *jB, float lrate, float vexp);
int Java_edu_berkeley_bid_CUMACH_word2vecNegFilt(BidmachJNIEnv *env, void *obj, int nrows,
                                                 int ncols, int nwords, int nwa, int nwb, void *jWA,
                                                 void *jWB, void *jA, void *jB, float lrate,
                                                 float vexp);
int Java_edu_berkeley_bid_CUMACH_word2vecEvalPos(BidmachJNIEnv *env, void *obj, int nrows,
                                                 int ncols, int shift, void *jW, void *jLB,
                                                 void *jUB, void *jA, void *jB, void *jRetval);
int Java_edu_berkeley_bid_CUMACH_word2vecEvalNeg(BidmachJNIEnv *env, void *obj, int nrows,
                                                 int ncols, int nwa, int nwb, void *jWA, void *jWB,
                                                 void *jA, void *jB, void *jRetval);

/* Binders of the whole-minibatch extension (part 3), for a CUMACH that declares
 *   native long w2vCreate(int dim, int nskip, int nneg, int nreuse, int vocabSize, float wexpt,
 *                         float wsample, float lrate, float texp, float vexp, int iflip, int eqPosNeg,
 *                         int permute, long seed, int ncols);            // 0 = refused
 *   native void w2vDestroy(long ctx);
 *   native int w2vInitModel(long ctx, Pointer A, Pointer B);
 *   native int w2vDobatch(long ctx, Pointer tokens, Pointer A, Pointer B, long pos, long batchId);
 *   native double w2vEvalbatch(long ctx, Pointer tokens, Pointer A, Pointer B, long batchId);  // NaN = error
 *   native int w2vLastError(long ctx);
 * Work goes to the calling thread's default stream, as with the five binders above. */
int64_t Java_edu_berkeley_bid_CUMACH_w2vCreate(BidmachJNIEnv *env, void *obj, int dim, int nskip, int nneg,
                                               int nreuse, int vocabSize, float wexpt, float wsample,
                                               float lrate, float texp, float vexp, int iflip,
                                               int eqPosNeg, int permute, int64_t seed, int ncols);
void Java_edu_berkeley_bid_CUMACH_w2vDestroy(BidmachJNIEnv *env, void *obj, int64_t ctx);
int Java_edu_berkeley_bid_CUMACH_w2vInitModel(BidmachJNIEnv *env, void *obj, int64_t ctx, void *jA,
                                              void *jB);
int Java_edu_berkeley_bid_CUMACH_w2vDobatch(BidmachJNIEnv *env, void *obj, int64_t ctx, void *jTokens,
                                            void *jA, void *jB, int64_t pos, int64_t batchId);
double Java_edu_berkeley_bid_CUMACH_w2vEvalbatch(BidmachJNIEnv *env, void *obj, int64_t ctx,
                                                 void *jTokens, void *jA, void *jB, int64_t batchId);
int Java_edu_berkeley_bid_CUMACH_w2vLastError(BidmachJNIEnv *env, void *obj, int64_t ctx);
#endif

/* ------------------------------------------------------------------------
 * Part 3 -- whole-minibatch extension (no counterpart among the reference's
 * native functions; it moves the body of Word2Vec.dobatch / evalbatch /
 * wordMats, networks/Word2Vec.scala:167-278, onto the device so that a
 * minibatch costs one call and no JVM-side matrix operations).
 * ---------------------------------------------------------------------- */

/* Same names, meaning and defaults as Word2Vec.Opts (networks/Word2Vec.scala:
 * 574-591) plus dim (models/Model.scala:537) and lrate/texp/vexp
 * (updaters/Grad.scala:242-243, updaters/ADAGrad.scala:158). */
typedef struct w2v_opts {
  int dim;          /* 256 */
  int nskip;        /* 5   */
  int nneg;         /* 5   */
  int nreuse;       /* 5   */
  int vocabSize;    /* 100000 */
  float wexpt;      /* 0.75  */
  float wsample;    /* 1e-4  */
  float lrate;      /* 1     */
  float texp;       /* 0.5   */
  float vexp;       /* 0.5   */
  int iflip;        /* 0: row 0 of the minibatch is the word id, row 1 the sentence id */
  int eqPosNeg;     /* 0: negatives use lrate / nneg */
  int permute;      /* how the pair list is shuffled (Word2Vec.scala:254-259 sorts it by random keys):
                       0: keyed bijection of the pair indices, no sort and no host synchronisation;
                       1: sort by random keys as the reference's GPU branch.  Keys given in
                       w2v_uniforms.permute always select the sort. */
  uint64_t seed;    /* seed of the built-in counter-based generator */
} w2v_opts;

typedef struct w2v_ctx w2v_ctx;

/* Optional explicit random inputs.  A null member is drawn from the built-in
 * Philox4x32-10 generator keyed by (opts.seed, batch counter); a non-null
 * member is used as given, which makes the preprocessing a deterministic map
 * that can be compared bit for bit with the CPU path.  All are device fp32:
 *   sample  [ncols]            subsampling draw   (Word2Vec.scala:221)
 *   window  [ncols]            window-size draw   (Word2Vec.scala:228)
 *   permute [2*nskip x ncols]  permutation keys, column-major (Word2Vec.scala:254)
 *   negs    [nneg x ngroups]   negative draws, at least nneg*(pairs/nreuse) (Word2Vec.scala:264) */
typedef struct w2v_uniforms {
  const float *sample;
  const float *window;
  const float *permute;
  const float *negs;
} w2v_uniforms;

void w2v_default_opts(w2v_opts *opts);

/* Allocates the per-minibatch work buffers for minibatches of exactly `ncols`
 * tokens on the current device.  Returns 1 for unsupported options. */
int w2v_create(const w2v_opts *opts, int ncols, w2v_ctx **out);
void w2v_destroy(w2v_ctx *ctx);

/* modelmats(0) = (U[0,1) - 0.5) / dim, modelmats(1) = 0 (Word2Vec.scala:113-117).
 * B receives modelmats(0) and A modelmats(1); both dim x vocabSize. */
int w2v_init_model(const w2v_opts *opts, float *A, float *B, void *stream);

/* Word2Vec.wordMats (Word2Vec.scala:214-278): subsampling, window bounds,
 * ordered context list, random permutation, negative ids.  `tokens` is the
 * 2 x ncols int32 minibatch, column-major.  Results stay in the context and
 * are read with w2v_buffers.  With the sorted permutation the call
 * synchronises `stream` once (the sort needs the pair count on the host); with
 * the keyed bijection it only enqueues work. */
int w2v_wordmats(w2v_ctx *ctx, const int *tokens, const w2v_uniforms *u, uint64_t batch_id,
                 void *stream);

typedef struct w2v_buffers_t {
  int *words, *lb, *ub;   /* int32[ncols]                                      */
  int *contexts;          /* int32[npairs] ordered list (centre asc, offset asc) */
  int *WB;                /* int32[nreuse x ngroups] permuted context words    */
  int *WA;                /* int32[nneg x ngroups] negative words              */
  int64_t npairs;
  int ngroups;
} w2v_buffers_t;
/* Waits until the counts of the latest wordmats have reached the host. */
int w2v_buffers(w2v_ctx *ctx, w2v_buffers_t *out);

/* Word2Vec.dobatch (Word2Vec.scala:167-190): learning rate
 * lrate * (pos/firstPos)^(-texp), wordMats, positive update, negative update
 * with lrate/nneg (or lrate when eqPosNeg).  `pos` is the learner's running
 * sample position; the first call fixes firstPos. */
int w2v_dobatch(w2v_ctx *ctx, const int *tokens, const w2v_uniforms *u, float *A, float *B,
                int64_t pos, uint64_t batch_id, void *stream);

/* Word2Vec.evalbatch (Word2Vec.scala:192-212): wordMats, then
 * score = (evalPos + evalNeg / nneg) / (nreuse * ngroups), written to
 * *score_host (0 when the minibatch yields no group).  Synchronises. */
int w2v_evalbatch(w2v_ctx *ctx, const int *tokens, const w2v_uniforms *u, const float *A,
                  const float *B, uint64_t batch_id, double *score_host, void *stream);

/* Model.dobatchg / evalbatchg (models/Model.scala:350-365): the same two calls
 * for a minibatch that still lives in host memory (pinned, for the copy to be
 * asynchronous).  The tokens are uploaded inside the call, on a copy stream of
 * the context and into one of two buffers, so the upload of one minibatch runs
 * beside the kernels of the one before.  dobatch_host returns when the number
 * of positive pairs of this minibatch is known (by then the upload is complete
 * and the host buffer may be reused); the update kernels finish in stream
 * order, as after w2v_dobatch.  evalbatch_host returns the score and
 * therefore synchronises.  A staged kernel that gave up waiting for its copies
 * is reported by the next w2v_evalbatch / w2v_evalbatch_host. */
int w2v_dobatch_host(w2v_ctx *ctx, const int *tokens_host, float *A, float *B, int64_t pos,
                     uint64_t batch_id, int64_t *npairs_host, void *stream);
int w2v_evalbatch_host(w2v_ctx *ctx, const int *tokens_host, const float *A, const float *B,
                       uint64_t batch_id, double *score_host, void *stream);

/* Second half of an overlapped model average (multi-GPU): the caller snapshots
 * its replica into `base`, averages the snapshots of all replicas into `avg`
 * with an all-reduce that runs beside the following minibatches, and then
 * folds the result into the live replica: theta += avg - base, elementwise over
 * n floats (n a multiple of 4, pointers 16-byte aligned; else 1 is returned).
 * With this the exchange of Word2Vec.mergeModelFn (networks/Word2Vec.scala:
 * 547-568) no longer stalls training. */
int w2v_apply_average(float *theta, const float *base, const float *avg, int64_t n, void *stream);

/* Optional phase timers, the counterpart of the reference's per-phase
 * `times/delays` bookkeeping (networks/Word2Vec.scala:77-92): when switched on,
 * CUDA events are recorded at the phase boundaries of every minibatch and the
 * durations summed.  prep = subsampling, bounds, pair list; permute = sort and
 * negative ids; pos/neg = the two update kernels; evalpos/evalneg = the two
 * scoring kernels.  pairs/groups are the summed counts of the timed batches. */
typedef struct w2v_timing {
  double prep_ms, permute_ms, pos_ms, neg_ms, evalpos_ms, evalneg_ms;
  int64_t train_batches, eval_batches;
  int64_t pairs, groups, eval_pairs, eval_groups;
} w2v_timing;
int w2v_set_timing(w2v_ctx *ctx, int on);
int w2v_get_timing(w2v_ctx *ctx, w2v_timing *out); /* synchronises the last stream used */

/* Diagnostic: the memory side of the negative kernels alone, on the columns of
 * the latest w2v_wordmats.  mode 0: a row of zeros is added to every row of
 * every column with the update kernel's atomic reductions (A and B keep their
 * values); mode 1: every row is read; mode 2: as mode 0 with one bulk
 * reduction (shared -> global, add.f32) per row in place of the per-lane
 * reductions.  The duration of the call's kernel is
 * what the memory system needs for the scatter (the gather) of one negative
 * update (scoring) launch: the bound bench.py --mode bound reports. */
int w2v_probe_rows(w2v_ctx *ctx, float *A, float *B, int mode, void *stream);

/* Number of kernels this library has launched in this process (all threads). */
long long w2v_launch_count(void);

/* -------------------------------------------------------------------------
 * Part 4.  Byte codecs of BIDMat's compressed matrix files (host code).  The
 * reference reads corpora ("*.imat.lz4", scripts/getw2vdata.ssc:44) and writes
 * checkpoints ("modelmat%02d.lz4", models/Model.scala:259) through BIDMat's
 * loadMat / saveMat over lz4-java's block stream; these are the LZ4 block codec
 * and the XXH32 checksum that container needs.  The container itself and the
 * matrix header are handled by the host-side reader (bidmach_b200/matio.py).
 * ---------------------------------------------------------------------- */
uint32_t bidmach_xxh32(const void *data, int64_t len, uint32_t seed);
int64_t bidmach_lz4_compress_bound(int64_t n);
/* Both return the number of bytes written to dst, or -1 (dst too small;
 * malformed input).  Neither touches memory outside the given ranges. */
int64_t bidmach_lz4_compress(const void *src, int64_t n, void *dst, int64_t cap);
int64_t bidmach_lz4_decompress(const void *src, int64_t n, void *dst, int64_t cap);

#ifdef __cplusplus
}
#endif
#endif
