/* Minimal stand-in for <jni.h>, for a syntax / signature check of skainet_b200/jvm/native/skainet_cuda_jni.c where
 * no JDK exists (tests/test_jvm_sources.py). It declares only the types and JNIEnv functions that shim uses, with the
 * argument lists the JNI specification gives them. Not a JNI implementation: nothing here can run. */
#ifndef STUB_JNI_H
#define STUB_JNI_H
#include <stdint.h>
typedef int32_t jint; typedef int64_t jlong; typedef int8_t jbyte; typedef uint8_t jboolean; typedef float jfloat;
typedef void* jobject; typedef jobject jstring; typedef jobject jarray;
typedef jarray jfloatArray; typedef jarray jbyteArray; typedef jarray jintArray; typedef jarray jlongArray;
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define JNI_ABORT 2
struct JNINativeInterface_;
typedef const struct JNINativeInterface_* JNIEnv;
struct JNINativeInterface_ {
    void* (*GetPrimitiveArrayCritical)(JNIEnv* env, jarray array, jboolean* isCopy);
    void (*ReleasePrimitiveArrayCritical)(JNIEnv* env, jarray array, void* carray, jint mode);
    void* (*GetDirectBufferAddress)(JNIEnv* env, jobject buf);
    jstring (*NewStringUTF)(JNIEnv* env, const char* utf);
};
#endif
