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

}  // extern "C"
