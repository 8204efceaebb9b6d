/*
 * Plain-pointer front end for the reference's own CPU Word2Vec kernels.
 *
 * Test infrastructure, not product code.  build_ref.py compiles this file
 * together with the UNMODIFIED reference source jni/src/BIDMach_CPUMACH.c
 * (read where it lies, never copied) into oracle/_ref/libw2vref.so.  The
 * reference functions expect a JNIEnv; the one handed over here treats every
 * "Java array" as the raw C pointer it already is.
 *
 * Exposed calls (thin forwards, one per reference function):
 *   ref_word2vecPos     -> Java_edu_berkeley_bid_CPUMACH_word2vecPos     (BIDMach_CPUMACH.c:10-78)
 *   ref_word2vecNeg     -> Java_edu_berkeley_bid_CPUMACH_word2vecNeg     (BIDMach_CPUMACH.c:186-264)
 *   ref_word2vecEvalPos -> Java_edu_berkeley_bid_CPUMACH_word2vecEvalPos (BIDMach_CPUMACH.c:368-427)
 *   ref_word2vecEvalNeg -> Java_edu_berkeley_bid_CPUMACH_word2vecEvalNeg (BIDMach_CPUMACH.c:429-483)
 *   ref_word2vecPosSlice -> Java_edu_berkeley_bid_CPUMACH_word2vecPosSlice (BIDMach_CPUMACH.c:90-184)
 *   ref_word2vecNegSlice -> Java_edu_berkeley_bid_CPUMACH_word2vecNegSlice (BIDMach_CPUMACH.c:267-366)
 *     (the model is a Java float[][]: matrix 2*m holds the context rows and 2*m+1 the centre
 *     rows of block m of maxCols words; here an array of plain pointers)
 * The two eval functions of the reference add their per-thread sums onto an
 * uninitialised local (BIDMach_CPUMACH.c:379,423 and :439,479), so their
 * return value is only informational; the eval oracle is the restatement of
 * the Scala code in w2v_oracle.c.
 */
#include <jni.h>
#include <omp.h>

static void *drv_get_critical(JNIEnv *env, jarray arr, jboolean *is_copy) {
  (void)env;
  if (is_copy) *is_copy = JNI_FALSE;
  return arr;
}

static void drv_release_critical(JNIEnv *env, jarray arr, void *carr, jint mode) {
  (void)env; (void)arr; (void)carr; (void)mode;
}

static jsize drv_array_length(JNIEnv *env, jarray arr) {
  (void)env;
  return ((stub_objarray *)arr)->count;
}

static jobject drv_object_element(JNIEnv *env, jobjectArray arr, jsize index) {
  (void)env;
  return ((stub_objarray *)arr)->elems[index];
}

static const struct stub_jni_table drv_table = {
  drv_get_critical, drv_release_critical, drv_array_length, drv_object_element
};

extern void Java_edu_berkeley_bid_CPUMACH_word2vecPos(
    JNIEnv *, jobject, jint, jint, jint, jintArray, jintArray, jintArray,
    jfloatArray, jfloatArray, jfloat, jfloat, jint);
extern void Java_edu_berkeley_bid_CPUMACH_word2vecNeg(
    JNIEnv *, jobject, jint, jint, jint, jint, jintArray, jintArray,
    jfloatArray, jfloatArray, jfloat, jfloat, jint);
extern jdouble Java_edu_berkeley_bid_CPUMACH_word2vecEvalPos(
    JNIEnv *, jobject, jint, jint, jint, jintArray, jintArray, jintArray,
    jfloatArray, jfloatArray, jint);
extern jdouble Java_edu_berkeley_bid_CPUMACH_word2vecEvalNeg(
    JNIEnv *, jobject, jint, jint, const jint, const jint, jintArray, jintArray,
    jfloatArray, jfloatArray, jint);

extern void Java_edu_berkeley_bid_CPUMACH_word2vecPosSlice(
    JNIEnv *, jobject, jint, jint, jint, jintArray, jintArray, jintArray, jobjectArray, jfloat, jfloat,
    jint, jint, jint, jint, jint, jint, jint);
extern void Java_edu_berkeley_bid_CPUMACH_word2vecNegSlice(
    JNIEnv *, jobject, jint, jint, jint, jint, jintArray, jintArray, jfloatArray, jfloat, jfloat,
    jint, jint, jint, jint, jint, jint, jint);

void ref_word2vecPosSlice(int nrows, int ncols, int skip, int *W, int *LB, int *UB, float **mats,
                          int nmats, float lrate, float vexp, int nthreads, int islice, int nslices,
                          int maxCols, int nHead, int dualMode, int doHead) {
  JNIEnv env = &drv_table;
  stub_objarray mm = {nmats, (void **)mats};
  Java_edu_berkeley_bid_CPUMACH_word2vecPosSlice(&env, 0, nrows, ncols, skip, W, LB, UB, &mm, lrate,
                                                 vexp, nthreads, islice, nslices, maxCols, nHead,
                                                 dualMode, doHead);
}

void ref_word2vecNegSlice(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB, float **mats,
                          int nmats, float lrate, float vexp, int nthreads, int islice, int nslices,
                          int maxCols, int nHead, int dualMode, int doHead) {
  JNIEnv env = &drv_table;
  stub_objarray mm = {nmats, (void **)mats};
  Java_edu_berkeley_bid_CPUMACH_word2vecNegSlice(&env, 0, nrows, ncols, nwa, nwb, WA, WB, &mm, lrate,
                                                 vexp, nthreads, islice, nslices, maxCols, nHead,
                                                 dualMode, doHead);
}

void ref_word2vecPos(int nrows, int ncols, int skip, int *W, int *LB, int *UB,
                     float *A, float *B, float lrate, float vexp, int nthreads) {
  JNIEnv env = &drv_table;
  Java_edu_berkeley_bid_CPUMACH_word2vecPos(&env, 0, nrows, ncols, skip, W, LB, UB,
                                            A, B, lrate, vexp, nthreads);
}

void ref_word2vecNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB,
                     float *A, float *B, float lrate, float vexp, int nthreads) {
  JNIEnv env = &drv_table;
  Java_edu_berkeley_bid_CPUMACH_word2vecNeg(&env, 0, nrows, ncols, nwa, nwb, WA, WB,
                                            A, B, lrate, vexp, nthreads);
}

double ref_word2vecEvalPos(int nrows, int ncols, int skip, int *W, int *LB, int *UB,
                           float *A, float *B, int nthreads) {
  JNIEnv env = &drv_table;
  return Java_edu_berkeley_bid_CPUMACH_word2vecEvalPos(&env, 0, nrows, ncols, skip,
                                                       W, LB, UB, A, B, nthreads);
}

double ref_word2vecEvalNeg(int nrows, int ncols, int nwa, int nwb, int *WA, int *WB,
                           float *A, float *B, int nthreads) {
  JNIEnv env = &drv_table;
  return Java_edu_berkeley_bid_CPUMACH_word2vecEvalNeg(&env, 0, nrows, ncols, nwa, nwb,
                                                       WA, WB, A, B, nthreads);
}

/* The reference runs its chunks under "#pragma omp parallel for" with as many chunks as
 * `nthreads`; how many of them run at once is OpenMP's decision (OMP_NUM_THREADS, which
 * launchers such as torch.distributed.run set to 1).  ref_set_threads fixes the team size
 * and returns the size of the team a parallel region then really gets. */
int ref_set_threads(int n) {
  int got = 0;
  if (n > 0) omp_set_num_threads(n);
#pragma omp parallel
  {
#pragma omp single
    got = omp_get_num_threads();
  }
  return got;
}
