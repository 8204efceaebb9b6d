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
 * jni/src/DNN127.cu:1417-1419).  A call borrows a few MB of scratch memory from
 * a per-device pool; the pool allocates (cudaMalloc) only while more calls are
 * in flight on that device than ever before, so a host with one thread per GPU
 * sees one allocation per GPU for the life of the process, however many
 * threads come and go.
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

/* Vocabulary slices: the device forms of the reference's multi-node CPU kernels.  The model of
 * slice `islice` of `nslices` holds the rows of the head (ids below nHead, present on every
 * slice) followed by the rows of the ids with id % nslices == islice, id at row
 * (id - nHead) / nslices + nHead (mapIndx, jni/src/BIDMach_CPUMACH.c:80-88); A and B are those
 * two matrices (one per side: the reference cuts them into Java arrays of maxCols words, device
 * memory needs no such cut).  W / WA / WB hold global word ids.  A pair is worked on when both
 * words have a row here and, unless doHead > 1, not both are head words; head rows are written
 * only when doHead > 0.  Rows must be a multiple of 4 floats and the matrices 16-byte aligned.
 *
 * word2vecPosSlice replaces CPUMACH.word2vecPosSlice (jni/src/BIDMach_CPUMACH.c:90-184; called
 * from networks/Word2Vec.scala:425), word2vecNegSlice replaces CPUMACH.word2vecNegSlice
 * (BIDMach_CPUMACH.c:267-366; Word2Vec.scala:459).  The two scoring functions replace
 * Word2Vec.evalPosCPUslice / evalNegCPUslice (Word2Vec.scala:1007-1068, 1134-1200): the sum over
 * the pairs whose two words both have a row on this slice. */
int word2vecPosSlice(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                     float lrate, float vexp, int islice, int nslices, int nHead, int doHead);
int word2vecNegSlice(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                     float lrate, float vexp, int islice, int nslices, int nHead, int doHead);
int word2vecEvalPosSlice(int nrows, int ncols, int shift, int *W, int *LB, int *UB, float *A, float *B,
                         float *Retval, int islice, int nslices, int nHead);
int word2vecEvalNegSlice(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float *A, float *B,
                         float *Retval, int islice, int nslices, int nHead);

/* No counterpart in the reference.  Same contract as word2vecEvalNeg, for
 * hosts that must not allocate device memory while they run (a JVM whose matrix
 * cache already owns the card, a process that froze its memory map): the
 * partial sums live in an array built into the library's device image (about
 * 64 KiB on every GPU that loads the library) instead of a buffer obtained with
 * cudaMalloc.  At most 2,097,152 columns per call; a larger ncols prints a
 * message and returns 1.  The first call on a device looks up the array's
 * device address (a runtime query, not an allocation); let that first call
 * happen before the process starts any stream capture on that device.  The
 * function waits for its kernel, like the launchers
 * above.  Calls on the same GPU share the array: do not let two of them run at
 * the same time. */
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
int Java_edu_berkeley_bid_CUMACH_w2vSetSlice(BidmachJNIEnv *env, void *obj, int64_t ctx, int islice,
                                             int nslices, int nHead, int doHead);

/* Binders of the vocabulary-slice launchers and of the model exchange (both further down in part
 * 1 and part 3): same argument lists with jcuda.Pointer objects in place of the device pointers.
 *   native int  word2vecPosSlice(..., int islice, int nslices, int nHead, int doHead);      etc.
 *   native long w2vCommInitAll(int ndev);   native long w2vCommOf(long comms, int i);
 *   native int  w2vAllreduceAvg(long comm, Pointer A, Pointer B, long nEach);
 *   native void w2vCommDestroyAll(long comms); */
int Java_edu_berkeley_bid_CUMACH_word2vecPosSlice(BidmachJNIEnv *env, void *obj, int nrows, int ncols,
                                                  int shift, void *jW, void *jLB, void *jUB, void *jA,
                                                  void *jB, float lrate, float vexp, int islice,
                                                  int nslices, int nHead, int doHead);
int Java_edu_berkeley_bid_CUMACH_word2vecNegSlice(BidmachJNIEnv *env, void *obj, int nrows, int ncols,
                                                  int nwa, int nwb, void *jWA, void *jWB, void *jA,
                                                  void *jB, float lrate, float vexp, int islice,
                                                  int nslices, int nHead, int doHead);
int Java_edu_berkeley_bid_CUMACH_word2vecEvalPosSlice(BidmachJNIEnv *env, void *obj, int nrows, int ncols,
                                                      int shift, void *jW, void *jLB, void *jUB, void *jA,
                                                      void *jB, void *jRetval, int islice, int nslices,
                                                      int nHead);
int Java_edu_berkeley_bid_CUMACH_word2vecEvalNegSlice(BidmachJNIEnv *env, void *obj, int nrows, int ncols,
                                                      int nwa, int nwb, void *jWA, void *jWB, void *jA,
                                                      void *jB, void *jRetval, int islice, int nslices,
                                                      int nHead);
int64_t Java_edu_berkeley_bid_CUMACH_w2vCommInitAll(BidmachJNIEnv *env, void *obj, int ndev);
int64_t Java_edu_berkeley_bid_CUMACH_w2vCommOf(BidmachJNIEnv *env, void *obj, int64_t comms, int i);
int Java_edu_berkeley_bid_CUMACH_w2vAllreduceAvg(BidmachJNIEnv *env, void *obj, int64_t comm, void *jA,
                                                 void *jB, int64_t nEach);
void Java_edu_berkeley_bid_CUMACH_w2vCommDestroyAll(BidmachJNIEnv *env, void *obj, int64_t comms);
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

/* ---- model exchange between replicas (multi-GPU) --------------------------
 * Replaces Word2Vec.mergeModelFn (networks/Word2Vec.scala:547-568), which
 * averages the model matrices of all GPUs through host-driven peer copies, and
 * ParLearner.syncmodels that calls it (Learner.scala:655).
 *
 * For a host with one thread per GPU in one process (the reference's ParLearner,
 * Learner.scala:589-655) or one process per GPU: a communicator per GPU, then
 * w2v_allreduce_avg on every replica at the same point of its minibatch
 * sequence.  NCCL (libnccl.so.2) is loaded at run time; without it these
 * return 2.  Other errors: 1 for bad arguments, a cudaError_t, or 2000 + the
 * ncclResult_t. */
typedef struct w2v_comm w2v_comm;
/* One process, ndev devices (null `devices` = 0..ndev-1): comms[i] belongs to
 * devices[i] and is to be used by the thread that drives that GPU. */
int w2v_comm_init_all(int ndev, const int *devices, w2v_comm **comms);
/* One process per GPU: rank 0 fills a 128-byte id with w2v_comm_unique_id and
 * hands it to the other ranks (any channel); every rank then calls
 * w2v_comm_init_rank with its device current. */
int w2v_comm_unique_id(void *id128);
int w2v_comm_init_rank(int nranks, int rank, const void *id128, w2v_comm **out);
/* Optional: registers the model buffer with the communicator, so that NCCL can
 * run the collective on the buffer in place (NVLink SHARP / zero copy) instead
 * of staging it.  The buffer stays the caller's. */
int w2v_comm_register(w2v_comm *comm, void *buf, int64_t bytes);
/* A[i] and B[i] (n_each floats each, device memory of the communicator's GPU)
 * become their mean over all replicas, in place, enqueued on `stream`.  When
 * B == A + n_each the two matrices travel as one collective. */
int w2v_allreduce_avg(w2v_comm *comm, float *A, float *B, int64_t n_each, void *stream);
void w2v_comm_destroy(w2v_comm *comm);

/* The same average without NCCL, for a buffer that is mapped on every replica's
 * GPU through an NVLink multicast address (symmetric memory of one process per
 * GPU): replica `rank` of `world` averages its 1/world slice of the n floats
 * with multimem.ld_reduce (the NVSwitch adds the replicas' values) and
 * multimem.st (the mean goes back to every replica).  `mc_base` is the
 * multicast address of the first float, 16-byte aligned, n a multiple of 4.
 * `blocks` limits the kernel to that many SMs (0 = all), so that it can run
 * beside the update kernels of the next minibatch.  The kernel waits for
 * nobody: the caller orders it after every replica's last update (a barrier or
 * any collective on the same stream) unless it accepts the relaxed form below.
 * Concurrent use: an update that lands on an element between the kernel's read
 * and its write of that element (a few microseconds) is overwritten by the
 * mean; updates before are averaged in, updates after are kept. */
int w2v_nvls_average(float *mc_base, int64_t n, int rank, int world, int blocks, void *stream);
/* The same with plain peer loads and stores: replicas_host[r] (a host array of `world` <= 8
 * device pointers) is replica r's address of the buffer as this GPU sees it (peer access or
 * symmetric memory), replicas_host[rank] the local one.  Moves fewer bytes over NVLink than the
 * multicast form for two or three replicas. */
int w2v_p2p_average(float *const *replicas_host, int64_t n, int rank, int world, int blocks, void *stream);

/* Word2Vec.Opts nSlices / iSlice / nHeadTerms / doHead (networks/Word2Vec.scala:586-590) for the
 * whole-minibatch calls: A and B given to w2v_dobatch / w2v_evalbatch then hold the rows of that
 * slice only (w2v_slice_rows of them), the minibatch still carries global ids.  The default is
 * the whole vocabulary (nslices 1). */
int w2v_set_slice(w2v_ctx *ctx, int islice, int nslices, int nHead, int doHead);
/* Rows of a slice's matrices: nHead + 1 + (vocabSize - nHead - 1) / nslices (Word2Vec.scala:106). */
int64_t w2v_slice_rows(int vocabSize, int nslices, int nHead);

/* Keeps `sms` SMs out of the grid of the negative update that the following
 * w2v_dobatch / w2v_dobatch_host calls launch (0 = use every SM again), so that
 * a kernel on another stream -- the overlapped w2v_nvls_average -- finds free
 * SMs while it runs (the negative update is bound by the L2's atomic throughput
 * and loses nothing measurable to a few SMs fewer). */
int w2v_reserve_sms(w2v_ctx *ctx, int sms);
/* Makes `stream` wait until the positive update of the latest w2v_dobatch / w2v_dobatch_host call
 * has finished (and with it everything of the minibatches before): the point from which an
 * exchange on another stream runs beside the negative update only. */
int w2v_wait_pos(w2v_ctx *ctx, void *stream);
/* The negative update of the next w2v_dobatch / w2v_dobatch_host call waits for `event` (a
 * cudaEvent_t, which must stay alive until that call; null withdraws it) before it starts, while
 * that call's preprocessing and positive update do not: an exchange that outlasts the negative
 * update it started beside finishes beside the next minibatch's first kernels. */
int w2v_wait_before_neg(w2v_ctx *ctx, void *event);

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
