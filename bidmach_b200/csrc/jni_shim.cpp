// JNI entry points of edu.berkeley.bid.CUMACH for the Word2Vec path.
//
// Replaces, with the same exported names and argument lists, the binders in
// jni/src/BIDMach_CUMACH.cpp:434-493 and JNI_OnLoad at :11-29.  Each binder
// unwraps its jcuda.Pointer arguments to device addresses and forwards to the
// C launcher of the same name.  A jcuda.Pointer's address is
// NativePointerObject.nativePointer + Pointer.byteOffset, and a null reference
// is a null pointer (jni/src/PointerUtils.cpp:353-363); the two field ids are
// looked up once in JNI_OnLoad (jni/src/PointerUtils.cpp:76-88).
#if defined(__has_include)
#if __has_include(<jni.h>)
#include <jni.h>
#define W2V_REAL_JNI 1
#endif
#endif
#ifndef W2V_REAL_JNI
#include "jni_min.h"
#endif

#include <cuda_runtime_api.h>

#define BIDMACH_B200_NO_JNI_DECLS
#include "../../include/bidmach_b200.h"

namespace {

jfieldID g_native_pointer = nullptr;  // jcuda.NativePointerObject.nativePointer : J
jfieldID g_byte_offset = nullptr;     // jcuda.Pointer.byteOffset : J

#ifdef W2V_REAL_JNI
inline jclass find_class(JNIEnv *env, const char *n) { return env->FindClass(n); }
inline jfieldID field_id(JNIEnv *env, jclass c, const char *n, const char *s) { return env->GetFieldID(c, n, s); }
inline jlong long_field(JNIEnv *env, jobject o, jfieldID f) { return env->GetLongField(o, f); }
inline jint get_env(JavaVM *vm, void **penv) { return vm->GetEnv(penv, JNI_VERSION_1_4); }
#else
inline jclass find_class(JNIEnv *env, const char *n) { return jni_FindClass(env, n); }
inline jfieldID field_id(JNIEnv *env, jclass c, const char *n, const char *s) { return jni_GetFieldID(env, c, n, s); }
inline jlong long_field(JNIEnv *env, jobject o, jfieldID f) { return jni_GetLongField(env, o, f); }
inline jint get_env(JavaVM *vm, void **penv) { return jvm_GetEnv(vm, penv, JNI_VERSION_1_4); }
#endif

int cache_field_ids(JNIEnv *env) {
  jclass npo = find_class(env, "jcuda/NativePointerObject");
  if (!npo) return JNI_ERR;
  g_native_pointer = field_id(env, npo, "nativePointer", "J");
  if (!g_native_pointer) return JNI_ERR;
  jclass ptr = find_class(env, "jcuda/Pointer");
  if (!ptr) return JNI_ERR;
  g_byte_offset = field_id(env, ptr, "byteOffset", "J");
  if (!g_byte_offset) return JNI_ERR;
  return JNI_OK;
}

inline void *device_address(JNIEnv *env, jobject pointer_object) {
  if (pointer_object == nullptr) return nullptr;
  jlong base = long_field(env, pointer_object, g_native_pointer);
  jlong off = long_field(env, pointer_object, g_byte_offset);
  return (void *)(intptr_t)(base + off);
}

}  // namespace

extern "C" {

JNIEXPORT jint JNICALL JNI_OnLoad(JavaVM *jvm, void *reserved) {
  (void)reserved;
  JNIEnv *env = nullptr;
  if (get_env(jvm, (void **)&env) != JNI_OK || env == nullptr) return JNI_ERR;
  if (cache_field_ids(env) != JNI_OK) return JNI_ERR;
  return JNI_VERSION_1_4;
}

// Test hook: the address the binders would pass on for this jcuda.Pointer.
JNIEXPORT void *bidmach_jni_device_address(JNIEnv *env, jobject pointer_object) {
  return device_address(env, pointer_object);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecPos(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint shift, jobject jW, jobject jLB,
    jobject jUB, jobject jA, jobject jB, jfloat lrate, jfloat vexp) {
  (void)obj;
  return word2vecPos(nrows, ncols, shift, (int *)device_address(env, jW),
                     (int *)device_address(env, jLB), (int *)device_address(env, jUB),
                     (float *)device_address(env, jA), (float *)device_address(env, jB), lrate,
                     vexp);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecNeg(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint nwa, jint nwb, jobject jWA, jobject jWB,
    jobject jA, jobject jB, jfloat lrate, jfloat vexp) {
  (void)obj;
  return word2vecNeg(nrows, ncols, nwa, nwb, (int *)device_address(env, jWA),
                     (int *)device_address(env, jWB), (float *)device_address(env, jA),
                     (float *)device_address(env, jB), lrate, vexp);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecNegFilt(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint nwords, jint nwa, jint nwb, jobject jWA,
    jobject jWB, jobject jA, jobject jB, jfloat lrate, jfloat vexp) {
  (void)obj;
  return word2vecNegFilt(nrows, ncols, nwords, nwa, nwb, (int *)device_address(env, jWA),
                         (int *)device_address(env, jWB), (float *)device_address(env, jA),
                         (float *)device_address(env, jB), lrate, vexp);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecEvalPos(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint shift, jobject jW, jobject jLB,
    jobject jUB, jobject jA, jobject jB, jobject jRetval) {
  (void)obj;
  return word2vecEvalPos(nrows, ncols, shift, (int *)device_address(env, jW),
                         (int *)device_address(env, jLB), (int *)device_address(env, jUB),
                         (float *)device_address(env, jA), (float *)device_address(env, jB),
                         (float *)device_address(env, jRetval));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecEvalNeg(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint nwa, jint nwb, jobject jWA, jobject jWB,
    jobject jA, jobject jB, jobject jRetval) {
  (void)obj;
  return word2vecEvalNeg(nrows, ncols, nwa, nwb, (int *)device_address(env, jWA),
                         (int *)device_address(env, jWB), (float *)device_address(env, jA),
                         (float *)device_address(env, jB), (float *)device_address(env, jRetval));
}

// ---------------------------------------------------------------------------
// Binders for the whole-minibatch extension (part 3 of the header), so that a
// JVM host needs nothing but the matching `native` declarations in
// edu.berkeley.bid.CUMACH:
//
//   public static native long   w2vCreate(int dim, int nskip, int nneg, int nreuse, int vocabSize,
//                                         float wexpt, float wsample, float lrate, float texp, float vexp,
//                                         int iflip, int eqPosNeg, int permute, long seed, int ncols);
//   public static native void   w2vDestroy(long ctx);
//   public static native int    w2vInitModel(long ctx, Pointer A, Pointer B);
//   public static native int    w2vDobatch(long ctx, Pointer tokens, Pointer A, Pointer B, long pos, long batchId);
//   public static native double w2vEvalbatch(long ctx, Pointer tokens, Pointer A, Pointer B, long batchId);
//   public static native int    w2vLastError(long ctx);
//
// The context handle travels as a long.  Work goes to the calling thread's
// default stream, as the five reference binders; w2vDobatch only enqueues,
// w2vEvalbatch returns the score (NaN after an error, whose code w2vLastError
// then reports).
// ---------------------------------------------------------------------------
namespace {
struct JniCtx {
  w2v_ctx *ctx;
  w2v_opts opts;
  int last_error;
};
void *const kPerThreadStream = (void *)cudaStreamPerThread;
}  // namespace

JNIEXPORT jlong JNICALL Java_edu_berkeley_bid_CUMACH_w2vCreate(
    JNIEnv *env, jobject obj, jint dim, jint nskip, jint nneg, jint nreuse, jint vocabSize, jfloat wexpt,
    jfloat wsample, jfloat lrate, jfloat texp, jfloat vexp, jint iflip, jint eqPosNeg, jint permute,
    jlong seed, jint ncols) {
  (void)env;
  (void)obj;
  JniCtx *h = new JniCtx();
  w2v_default_opts(&h->opts);
  h->opts.dim = dim;
  h->opts.nskip = nskip;
  h->opts.nneg = nneg;
  h->opts.nreuse = nreuse;
  h->opts.vocabSize = vocabSize;
  h->opts.wexpt = wexpt;
  h->opts.wsample = wsample;
  h->opts.lrate = lrate;
  h->opts.texp = texp;
  h->opts.vexp = vexp;
  h->opts.iflip = iflip;
  h->opts.eqPosNeg = eqPosNeg;
  h->opts.permute = permute;
  h->opts.seed = (uint64_t)seed;
  h->last_error = w2v_create(&h->opts, ncols, &h->ctx);
  if (h->last_error) {
    delete h;
    return 0;
  }
  return (jlong)(intptr_t)h;
}

JNIEXPORT void JNICALL Java_edu_berkeley_bid_CUMACH_w2vDestroy(JNIEnv *env, jobject obj, jlong handle) {
  (void)env;
  (void)obj;
  JniCtx *h = (JniCtx *)(intptr_t)handle;
  if (!h) return;
  w2v_destroy(h->ctx);
  delete h;
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_w2vInitModel(JNIEnv *env, jobject obj, jlong handle,
                                                                 jobject jA, jobject jB) {
  (void)obj;
  JniCtx *h = (JniCtx *)(intptr_t)handle;
  if (!h) return 1;
  return h->last_error = w2v_init_model(&h->opts, (float *)device_address(env, jA),
                                        (float *)device_address(env, jB), kPerThreadStream);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_w2vDobatch(JNIEnv *env, jobject obj, jlong handle,
                                                               jobject jTokens, jobject jA, jobject jB,
                                                               jlong pos, jlong batchId) {
  (void)obj;
  JniCtx *h = (JniCtx *)(intptr_t)handle;
  if (!h) return 1;
  return h->last_error = w2v_dobatch(h->ctx, (const int *)device_address(env, jTokens), nullptr,
                                     (float *)device_address(env, jA), (float *)device_address(env, jB),
                                     pos, (uint64_t)batchId, kPerThreadStream);
}

JNIEXPORT jdouble JNICALL Java_edu_berkeley_bid_CUMACH_w2vEvalbatch(JNIEnv *env, jobject obj, jlong handle,
                                                                    jobject jTokens, jobject jA, jobject jB,
                                                                    jlong batchId) {
  (void)obj;
  JniCtx *h = (JniCtx *)(intptr_t)handle;
  double score = 0.0;
  const double nan = __builtin_nan("");
  if (!h) return nan;
  h->last_error = w2v_evalbatch(h->ctx, (const int *)device_address(env, jTokens), nullptr,
                                (const float *)device_address(env, jA), (const float *)device_address(env, jB),
                                (uint64_t)batchId, &score, kPerThreadStream);
  return h->last_error ? nan : score;
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_w2vLastError(JNIEnv *env, jobject obj, jlong handle) {
  (void)env;
  (void)obj;
  JniCtx *h = (JniCtx *)(intptr_t)handle;
  return h ? h->last_error : 1;
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_w2vSetSlice(JNIEnv *env, jobject obj, jlong handle,
                                                                jint islice, jint nslices, jint nHead,
                                                                jint doHead) {
  (void)env;
  (void)obj;
  JniCtx *h = (JniCtx *)(intptr_t)handle;
  if (!h) return 1;
  return h->last_error = w2v_set_slice(h->ctx, islice, nslices, nHead, doHead);
}

// ---------------------------------------------------------------------------
// Binders of the vocabulary-slice launchers, for a CUMACH that declares
//   native int word2vecPosSlice(int nrows, int ncols, int shift, Pointer W, Pointer LB, Pointer UB, Pointer A,
//                               Pointer B, float lrate, float vexp, int islice, int nslices, int nHead, int doHead);
//   native int word2vecNegSlice(int nrows, int ncols, int nwa, int nwb, Pointer WA, Pointer WB, Pointer A,
//                               Pointer B, float lrate, float vexp, int islice, int nslices, int nHead, int doHead);
//   native int word2vecEvalPosSlice(..., Pointer retVal, int islice, int nslices, int nHead);
//   native int word2vecEvalNegSlice(..., Pointer retVal, int islice, int nslices, int nHead);
// (the device forms of CPUMACH.word2vecPosSlice / word2vecNegSlice, jni/src/BIDMach_CPUMACH.c:90-184, 267-366).
// ---------------------------------------------------------------------------
JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecPosSlice(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint shift, jobject jW, jobject jLB, jobject jUB,
    jobject jA, jobject jB, jfloat lrate, jfloat vexp, jint islice, jint nslices, jint nHead, jint doHead) {
  (void)obj;
  return word2vecPosSlice(nrows, ncols, shift, (int *)device_address(env, jW), (int *)device_address(env, jLB),
                          (int *)device_address(env, jUB), (float *)device_address(env, jA),
                          (float *)device_address(env, jB), lrate, vexp, islice, nslices, nHead, doHead);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecNegSlice(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint nwa, jint nwb, jobject jWA, jobject jWB,
    jobject jA, jobject jB, jfloat lrate, jfloat vexp, jint islice, jint nslices, jint nHead, jint doHead) {
  (void)obj;
  return word2vecNegSlice(nrows, ncols, nwa, nwb, (int *)device_address(env, jWA),
                          (int *)device_address(env, jWB), (float *)device_address(env, jA),
                          (float *)device_address(env, jB), lrate, vexp, islice, nslices, nHead, doHead);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecEvalPosSlice(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint shift, jobject jW, jobject jLB, jobject jUB,
    jobject jA, jobject jB, jobject jRetval, jint islice, jint nslices, jint nHead) {
  (void)obj;
  return word2vecEvalPosSlice(nrows, ncols, shift, (int *)device_address(env, jW),
                              (int *)device_address(env, jLB), (int *)device_address(env, jUB),
                              (float *)device_address(env, jA), (float *)device_address(env, jB),
                              (float *)device_address(env, jRetval), islice, nslices, nHead);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_word2vecEvalNegSlice(
    JNIEnv *env, jobject obj, jint nrows, jint ncols, jint nwa, jint nwb, jobject jWA, jobject jWB,
    jobject jA, jobject jB, jobject jRetval, jint islice, jint nslices, jint nHead) {
  (void)obj;
  return word2vecEvalNegSlice(nrows, ncols, nwa, nwb, (int *)device_address(env, jWA),
                              (int *)device_address(env, jWB), (float *)device_address(env, jA),
                              (float *)device_address(env, jB), (float *)device_address(env, jRetval), islice,
                              nslices, nHead);
}

// ---------------------------------------------------------------------------
// Binders of the model exchange, for a ParLearner with one thread per GPU:
//   native long w2vCommInitAll(int ndev);             // devices 0..ndev-1; 0 = failed
//   native long w2vCommOf(long comms, int i);         // the communicator of device i
//   native int  w2vAllreduceAvg(long comm, Pointer A, Pointer B, long nEach);   // thread i, its own matrices
//   native void w2vCommDestroyAll(long comms);
// w2vAllreduceAvg enqueues on the calling thread's default stream and returns; the next launcher
// call of that thread runs after it in stream order.
// ---------------------------------------------------------------------------
namespace {
struct JniComms {
  int ndev;
  w2v_comm *comm[64];
};
}  // namespace

JNIEXPORT jlong JNICALL Java_edu_berkeley_bid_CUMACH_w2vCommInitAll(JNIEnv *env, jobject obj, jint ndev) {
  (void)env;
  (void)obj;
  if (ndev < 1 || ndev > 64) return 0;
  JniComms *set = new JniComms();
  set->ndev = ndev;
  if (w2v_comm_init_all(ndev, nullptr, set->comm) != 0) {
    delete set;
    return 0;
  }
  return (jlong)(intptr_t)set;
}

JNIEXPORT jlong JNICALL Java_edu_berkeley_bid_CUMACH_w2vCommOf(JNIEnv *env, jobject obj, jlong comms, jint i) {
  (void)env;
  (void)obj;
  JniComms *set = (JniComms *)(intptr_t)comms;
  if (!set || i < 0 || i >= set->ndev) return 0;
  return (jlong)(intptr_t)set->comm[i];
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMACH_w2vAllreduceAvg(JNIEnv *env, jobject obj, jlong comm,
                                                                    jobject jA, jobject jB, jlong nEach) {
  (void)obj;
  return w2v_allreduce_avg((w2v_comm *)(intptr_t)comm, (float *)device_address(env, jA),
                           (float *)device_address(env, jB), nEach, kPerThreadStream);
}

JNIEXPORT void JNICALL Java_edu_berkeley_bid_CUMACH_w2vCommDestroyAll(JNIEnv *env, jobject obj, jlong comms) {
  (void)env;
  (void)obj;
  JniComms *set = (JniComms *)(intptr_t)comms;
  if (!set) return;
  for (int i = 0; i < set->ndev; i++) w2v_comm_destroy(set->comm[i]);
  delete set;
}

}  // extern "C"
