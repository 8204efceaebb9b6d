/*
 * Stand-in <jni.h> used ONLY to compile the reference's CPU kernels
 * (jni/src/BIDMach_CPUMACH.c) into the test oracle without a JDK.
 *
 * Test infrastructure, not product code.  It is not layout-compatible with a
 * real JVM: "arrays" are raw C pointers, and the JNIEnv only carries the four
 * calls that file makes (GetPrimitiveArrayCritical, its Release twin,
 * GetArrayLength, GetObjectArrayElement).  Object arrays (float[][] in the
 * slice kernels) are a {count, elements} record, see stub_objarray.
 */
#ifndef ORACLE_STUB_JNI_H
#define ORACLE_STUB_JNI_H

#include <stddef.h>
#include <stdarg.h>
#include <stdio.h> /* a JDK jni.h pulls this in; the reference relies on it */

typedef int jint;
typedef long long jlong;
typedef float jfloat;
typedef double jdouble;
typedef unsigned char jboolean;
typedef int jsize;

typedef void *jobject;
typedef jobject jclass;
typedef jobject jarray;
typedef jarray jintArray;
typedef jarray jfloatArray;
typedef jarray jdoubleArray;
typedef jarray jlongArray;
typedef jarray jobjectArray;

#define JNI_FALSE 0
#define JNI_TRUE 1
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL

typedef struct stub_objarray {
  jsize count;
  void **elems;
} stub_objarray;

struct stub_jni_table;
typedef const struct stub_jni_table *JNIEnv;

struct stub_jni_table {
  void *(*GetPrimitiveArrayCritical)(JNIEnv *env, jarray arr, jboolean *is_copy);
  void (*ReleasePrimitiveArrayCritical)(JNIEnv *env, jarray arr, void *carr, jint mode);
  jsize (*GetArrayLength)(JNIEnv *env, jarray arr);
  jobject (*GetObjectArrayElement)(JNIEnv *env, jobjectArray arr, jsize index);
};

#endif
