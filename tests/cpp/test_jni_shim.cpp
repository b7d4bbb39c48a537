// Drives the JNI shim (systemds_b200/csrc/cla_jni.cpp) against the fake JVM of jni_stub/jni.h: registers one group of
// every kind through the Java_..._CLANative_* entry points and checks that no JNI call was made while an array was
// pinned, that a null column array is refused, and that the handle reports the registered shape. No GPU is needed:
// registration is host-side work.
#include <jni.h>
#include <stdio.h>
#include <vector>
#include "../../include/systemds_cla.h"

#define JFN(name) Java_org_apache_sysds_runtime_compress_lib_CLANative_##name
extern "C" {
jlong JFN(create)(JNIEnv*, jclass, jint, jint, jboolean);
jlong JFN(destroy)(JNIEnv*, jclass, jlong);
jstring JFN(lastError)(JNIEnv*, jclass);
jlong JFN(addDDC)(JNIEnv*, jclass, jlong, jintArray, jdoubleArray, jint, jint, jarray, jbyteArray, jlong);
jlong JFN(addSDC)(JNIEnv*, jclass, jlong, jintArray, jdoubleArray, jint, jdoubleArray, jint, jint, jint, jarray, jlong, jint,
                  jarray, jbyteArray);
jlong JFN(addRLE)(JNIEnv*, jclass, jlong, jintArray, jdoubleArray, jint, jintArray, jcharArray);
jlong JFN(addOLE)(JNIEnv*, jclass, jlong, jintArray, jdoubleArray, jint, jintArray, jcharArray);
jlong JFN(addUncompressed)(JNIEnv*, jclass, jlong, jintArray, jdoubleArray);
jlong JFN(addConst)(JNIEnv*, jclass, jlong, jintArray, jdoubleArray);
jlong JFN(addEmpty)(JNIEnv*, jclass, jlong, jintArray);
jlong JFN(readBlock)(JNIEnv*, jclass, jbyteArray);
}

template <class T>
static FakeArray arr(std::vector<T>& v) { return FakeArray{v.data(), (jsize)v.size()}; }

int main() {
  JNIEnv env;
  const int nRows = 8;
  int fails = 0;
  auto expect = [&](bool ok, const char* what) {
    if (!ok) {
      printf("FAIL %s (%s)\n", what, JFN(lastError)(&env, nullptr));
      fails++;
    }
  };
  const jlong h = JFN(create)(&env, nullptr, nRows, 7, 0);
  expect(h > 0, "create");
  std::vector<int32_t> c0{0}, c1{1}, c2{2}, c3{3}, c45{4, 5}, c6{6};
  std::vector<double> d3{1.0, 2.0, 3.0}, d1{5.0}, dense(nRows * 2, 0.5), def{0.25};
  std::vector<uint8_t> map{0, 1, 2, 0, 1, 2, 0, 1}, sdcMap{0, 2}, offs{3};
  std::vector<int32_t> ptr{0, 2, 2, 2};
  std::vector<uint16_t> rle{1, 3}, ole{2, 0, 5};
  FakeArray a0 = arr(c0), a1 = arr(c1), a2 = arr(c2), a3 = arr(c3), a45 = arr(c45), a6 = arr(c6);
  FakeArray ad3 = arr(d3), ad1 = arr(d1), adense = arr(dense), adef = arr(def), amap = arr(map), asm_ = arr(sdcMap),
            aoff = arr(offs), aptr = arr(ptr), arle = arr(rle);
  std::vector<int32_t> optr{0, 3, 3, 3};
  FakeArray aoptr = arr(optr), aole = arr(ole);
  expect(JFN(addDDC)(&env, nullptr, h, &a0, &ad3, 3, CLA_MAP_UBYTE, &amap, nullptr, nRows) == 0, "addDDC");
  expect(JFN(addSDC)(&env, nullptr, h, &a1, &ad3, 3, &adef, CLA_OFF_BYTE, 2, 5, &aoff, 2, CLA_MAP_UBYTE, &asm_, nullptr) == 1,
         "addSDC");
  expect(JFN(addRLE)(&env, nullptr, h, &a2, &ad3, 3, &aptr, &arle) == 2, "addRLE");
  expect(JFN(addOLE)(&env, nullptr, h, &a3, &ad3, 3, &aoptr, &aole) == 3, "addOLE");
  expect(JFN(addUncompressed)(&env, nullptr, h, &a45, &adense) == 4, "addUncompressed");
  expect(JFN(addConst)(&env, nullptr, h, &a6, &ad1) == 5, "addConst");
  expect(JFN(addEmpty)(&env, nullptr, h, &a6) == 6, "addEmpty");
  // a null column array is an argument error, not a crash
  expect(JFN(addDDC)(&env, nullptr, h, nullptr, &ad3, 3, CLA_MAP_UBYTE, &amap, nullptr, nRows) == CLA_ERR_BAD_ARG, "addDDC(null cols)");
  expect(JFN(addEmpty)(&env, nullptr, h, nullptr) == CLA_ERR_BAD_ARG, "addEmpty(null cols)");
  std::vector<uint8_t> junk{1, 2, 3};
  FakeArray ajunk = arr(junk);
  expect(JFN(readBlock)(&env, nullptr, &ajunk) < 0, "readBlock(truncated)");
  cla_stats st;
  expect(cla_stats_get(h, &st) == CLA_OK && st.n_rows == nRows && st.n_cols == 7 && st.n_groups == 7, "stats after registration");
  expect(JFN(destroy)(&env, nullptr, h) == CLA_OK, "destroy");
  expect(env.violations == 0, "no JNI call inside a critical region");
  expect(env.nullDereferences == 0, "GetArrayLength never sees null");
  expect(env.pinned == 0, "every pinned array released");
  printf(fails ? "JNI SHIM: %d FAILURES\n" : "JNI SHIM OK\n", fails);
  return fails ? 1 : 0;
}
