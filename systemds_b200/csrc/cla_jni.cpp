// JNI shim: one native method per C-ABI call, for a Java class
// org.apache.sysds.runtime.compress.lib.CLANative that declares the same methods as `static native`.
// Built only where <jni.h> exists (the reference does the same for its native libraries); it adds no logic:
// arrays are pinned with GetPrimitiveArrayCritical and released JNI_ABORT for inputs / 0 for outputs, the
// convention of the reference's BLAS bridge (src/main/cpp/systemds.cpp:38-56). Return values pass through:
// >= 0 is the number of non-zeros of the result (or a handle / group index), < 0 a CLA_ERR_* code that the
// Java side turns into a DMLCompressionException with the text of cla_last_error.
//
// No JNI function may be called between GetPrimitiveArrayCritical and its release, so every method reads the
// array lengths it needs first and pins afterwards. The product methods keep their operands pinned for the
// length of the GPU call, as the reference's dmmdd / tsmm bridge does for its BLAS call: the collector is held
// off for that long (milliseconds at the benchmark sizes).
#include <jni.h>
#include "../../include/systemds_cla.h"

namespace {
struct In {  // pinned input array (may be null)
  JNIEnv* e;
  jarray a;
  void* p;
  In(JNIEnv* env, jarray arr) : e(env), a(arr), p(arr ? env->GetPrimitiveArrayCritical(arr, nullptr) : nullptr) {}
  ~In() { if (a) e->ReleasePrimitiveArrayCritical(a, p, JNI_ABORT); }
};
struct Out {  // pinned output array, contents copied back
  JNIEnv* e;
  jarray a;
  void* p;
  Out(JNIEnv* env, jarray arr) : e(env), a(arr), p(arr ? env->GetPrimitiveArrayCritical(arr, nullptr) : nullptr) {}
  ~Out() { if (a) e->ReleasePrimitiveArrayCritical(a, p, 0); }
};
}  // namespace

#define JFN(ret, name) extern "C" JNIEXPORT ret JNICALL Java_org_apache_sysds_runtime_compress_lib_CLANative_##name

JFN(jlong, create)(JNIEnv*, jclass, jint nRows, jint nCols, jboolean overlapping) {
  return cla_create(nRows, nCols, overlapping ? 1 : 0);
}
// the serialized block (CompressedMatrixBlock.write into a byte[]) in one call instead of one call per group
JFN(jlong, readBlock)(JNIEnv* env, jclass, jbyteArray bytes) {
  const jint len = bytes ? env->GetArrayLength(bytes) : 0;  // before pinning: no JNI calls inside a critical region
  In b(env, bytes);
  return cla_read_block((const uint8_t*)b.p, len, nullptr, nullptr);
}
JFN(jlong, destroy)(JNIEnv*, jclass, jlong h) { return cla_destroy(h); }
JFN(jlong, finalizeUpload)(JNIEnv*, jclass, jlong h, jint device) { return cla_finalize(h, device); }
JFN(jstring, lastError)(JNIEnv* env, jclass) {
  char buf[1024];
  cla_last_error(buf, sizeof(buf));
  return env->NewStringUTF(buf);
}

#define NEED_COLS(cols)                    \
  if (!cols) return CLA_ERR_BAD_ARG;      \
  const jint gCols = env->GetArrayLength(cols) /* before any array is pinned */

JFN(jlong, addDDC)(JNIEnv* env, jclass, jlong h, jintArray cols, jdoubleArray dict, jint nVals, jint mapType,
                   jarray map, jbyteArray mapHi, jlong mapSize) {
  NEED_COLS(cols);
  In c(env, cols), d(env, dict), m(env, map), mh(env, mapHi);
  return cla_add_group_ddc(h, (const int32_t*)c.p, gCols, (const double*)d.p, nVals, mapType, m.p, mh.p, mapSize);
}
JFN(jlong, addSDC)(JNIEnv* env, jclass, jlong h, jintArray cols, jdoubleArray dict, jint nVals, jdoubleArray def,
                   jint offType, jint first, jint last, jarray offData, jlong nOffsets, jint mapType, jarray map,
                   jbyteArray mapHi) {
  NEED_COLS(cols);
  const jlong offLen = offData ? env->GetArrayLength(offData) : 0;
  In c(env, cols), d(env, dict), df(env, def), o(env, offData), m(env, map), mh(env, mapHi);
  return cla_add_group_sdc(h, (const int32_t*)c.p, gCols, (const double*)d.p, nVals,
                           (const double*)df.p, offType, first, last, o.p, offLen, nOffsets, mapType, m.p, mh.p);
}
JFN(jlong, addRLE)(JNIEnv* env, jclass, jlong h, jintArray cols, jdoubleArray dict, jint nVals, jintArray ptr,
                   jcharArray data) {
  NEED_COLS(cols);
  const jlong dataLen = data ? env->GetArrayLength(data) : 0;
  In c(env, cols), d(env, dict), p(env, ptr), dt(env, data);
  return cla_add_group_rle(h, (const int32_t*)c.p, gCols, (const double*)d.p, nVals, (const int32_t*)p.p,
                           (const uint16_t*)dt.p, dataLen);
}
JFN(jlong, addOLE)(JNIEnv* env, jclass, jlong h, jintArray cols, jdoubleArray dict, jint nVals, jintArray ptr,
                   jcharArray data) {
  NEED_COLS(cols);
  const jlong dataLen = data ? env->GetArrayLength(data) : 0;
  In c(env, cols), d(env, dict), p(env, ptr), dt(env, data);
  return cla_add_group_ole(h, (const int32_t*)c.p, gCols, (const double*)d.p, nVals, (const int32_t*)p.p,
                           (const uint16_t*)dt.p, dataLen);
}
JFN(jlong, addUncompressed)(JNIEnv* env, jclass, jlong h, jintArray cols, jdoubleArray values) {
  NEED_COLS(cols);
  In c(env, cols), v(env, values);
  return cla_add_group_uncompressed(h, (const int32_t*)c.p, gCols, (const double*)v.p);
}
JFN(jlong, addConst)(JNIEnv* env, jclass, jlong h, jintArray cols, jdoubleArray tuple) {
  NEED_COLS(cols);
  In c(env, cols), t(env, tuple);
  return cla_add_group_const(h, (const int32_t*)c.p, gCols, (const double*)t.p);
}
JFN(jlong, addEmpty)(JNIEnv* env, jclass, jlong h, jintArray cols) {
  NEED_COLS(cols);
  In c(env, cols);
  return cla_add_group_empty(h, (const int32_t*)c.p, gCols);
}

JFN(jlong, rmm)(JNIEnv* env, jclass, jlong h, jdoubleArray V, jint vRows, jint vCols, jdoubleArray out) {
  In v(env, V);
  Out o(env, out);
  return cla_rmm(h, (const double*)v.p, vRows, vCols, (double*)o.p);
}
// X %*% V kept compressed (CLALibRightMultBy.rightMultByMatrix with allowOverlap): returns the handle of the new block
JFN(jlong, rmmOverlapping)(JNIEnv* env, jclass, jlong h, jdoubleArray V, jint vRows, jint vCols) {
  In v(env, V);
  return cla_rmm_overlapping(h, (const double*)v.p, vRows, vCols);
}
JFN(jlong, lmm)(JNIEnv* env, jclass, jlong h, jdoubleArray Yt, jint yRows, jdoubleArray out) {
  In y(env, Yt);
  Out o(env, out);
  return cla_lmm(h, (const double*)y.p, yRows, (double*)o.p);
}
JFN(jlong, tsmm)(JNIEnv* env, jclass, jlong h, jdoubleArray out) {
  Out o(env, out);
  return cla_tsmm(h, (double*)o.p);
}
JFN(jlong, tmm)(JNIEnv* env, jclass, jlong left, jlong right, jdoubleArray out) {
  Out o(env, out);
  return cla_tmm(left, right, (double*)o.p);
}
JFN(jlong, mmchain)(JNIEnv* env, jclass, jlong h, jdoubleArray v, jdoubleArray w, jint ctype, jdoubleArray out) {
  In vv(env, v), ww(env, w);
  Out o(env, out);
  return cla_mmchain(h, (const double*)vv.p, (const double*)ww.p, ctype, (double*)o.p);
}
JFN(jlong, unaryAgg)(JNIEnv* env, jclass, jlong h, jint op, jdoubleArray out) {
  Out o(env, out);
  return cla_unary_agg(h, op, (double*)o.p);
}
JFN(jlong, decompress)(JNIEnv* env, jclass, jlong h, jdoubleArray out) {
  Out o(env, out);
  return cla_decompress(h, (double*)o.p);
}
