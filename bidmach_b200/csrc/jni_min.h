// The few pieces of the Java Native Interface the CUMACH shim needs, for
// machines without a JDK.  Slot numbers are those of the JNI specification's
// function tables ("JNI Functions", Interface Function Table; "The Invocation
// API", JNIInvokeInterface); a JVM hands out tables with exactly this layout,
// so calling through the numbered slots is binary-compatible with <jni.h>.
// When a real <jni.h> is on the include path the shim uses that instead.
#pragma once

#include <stdint.h>

typedef int32_t jint;
typedef int64_t jlong;
typedef float jfloat;
typedef double jdouble;
typedef void *jobject;
typedef jobject jclass;
typedef void *jfieldID;

#define JNI_OK 0
#define JNI_ERR (-1)
#define JNI_VERSION_1_4 0x00010004
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL

// JNIEnv is a pointer to a table of function pointers.
typedef void *const *JNIEnvTable;
typedef JNIEnvTable JNIEnv;  // code receives JNIEnv*
typedef void *const *JavaVMTable;
typedef JavaVMTable JavaVM;  // code receives JavaVM*

enum {
  kJniFindClass = 6,
  kJniExceptionClear = 17,
  kJniNewGlobalRef = 21,
  kJniDeleteLocalRef = 23,
  kJniGetFieldID = 94,
  kJniGetLongField = 101,
  kJniExceptionCheck = 228,
  kJvmGetEnv = 6,
};

static inline jclass jni_FindClass(JNIEnv *env, const char *name) {
  return ((jclass(*)(JNIEnv *, const char *))(*env)[kJniFindClass])(env, name);
}
static inline jfieldID jni_GetFieldID(JNIEnv *env, jclass cls, const char *name, const char *sig) {
  return ((jfieldID(*)(JNIEnv *, jclass, const char *, const char *))(*env)[kJniGetFieldID])(
      env, cls, name, sig);
}
static inline jlong jni_GetLongField(JNIEnv *env, jobject obj, jfieldID fid) {
  return ((jlong(*)(JNIEnv *, jobject, jfieldID))(*env)[kJniGetLongField])(env, obj, fid);
}
static inline void jni_DeleteLocalRef(JNIEnv *env, jobject obj) {
  ((void (*)(JNIEnv *, jobject))(*env)[kJniDeleteLocalRef])(env, obj);
}
static inline jint jvm_GetEnv(JavaVM *vm, void **penv, jint version) {
  return ((jint(*)(JavaVM *, void **, jint))(*vm)[kJvmGetEnv])(vm, penv, version);
}
