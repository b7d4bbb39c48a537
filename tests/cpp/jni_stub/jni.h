// Stand-in for the JDK's <jni.h>, for machines without a JDK: just enough declarations to compile
// systemds_b200/csrc/cla_jni.cpp and to run its entry points against a fake JVM in tests/cpp/test_jni_shim.cpp.
// The fake environment records whether a JNI call is made while an array is pinned by
// GetPrimitiveArrayCritical, which the JNI specification forbids.
#pragma once
#include <stdint.h>
#include <string.h>

typedef int32_t jint;
typedef int64_t jlong;
typedef uint8_t jboolean;
typedef int32_t jsize;
struct FakeArray {
  void* data;
  jsize length;
};
typedef FakeArray* jobject;
typedef jobject jclass;
typedef jobject jarray;
typedef jarray jintArray;
typedef jarray jdoubleArray;
typedef jarray jbyteArray;
typedef jarray jcharArray;
typedef const char* jstring;
#define JNIEXPORT
#define JNICALL
#define JNI_ABORT 2

struct JNIEnv {
  int pinned = 0;            // arrays currently inside a critical region
  int violations = 0;        // JNI calls made while pinned > 0
  int nullDereferences = 0;  // GetArrayLength(NULL)
  char text[1024] = {0};
  void* GetPrimitiveArrayCritical(jarray a, void*) {
    pinned++;
    return a->data;
  }
  void ReleasePrimitiveArrayCritical(jarray, void*, int) { pinned--; }
  jsize GetArrayLength(jarray a) {
    if (pinned > 0) violations++;
    if (!a) {
      nullDereferences++;
      return 0;
    }
    return a->length;
  }
  jstring NewStringUTF(const char* s) {
    if (pinned > 0) violations++;
    strncpy(text, s, sizeof(text) - 1);
    return text;
  }
};
