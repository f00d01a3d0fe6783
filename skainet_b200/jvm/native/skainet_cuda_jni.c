/*
 * JNI shim over libskainet_cuda.so (include/skainet_cuda.h) for the Kotlin side of skainet-backend-cuda.
 *
 * UNVERIFIED SOURCE: no JDK (jni.h) exists where this library is built and tested, so this file has not been
 * compiled against a real JNI header; tests/test_jvm_sources.py compiles it against a minimal stand-in header to
 * catch syntax and signature slips. Everything numeric is verified through the same C ABI from Python.
 *
 * Pattern: skainet-backends/skainet-backend-jni-cpu/native/skainet_jni.c:10-31,146-181 — one function per kernel,
 * method names without underscores, GetPrimitiveArrayCritical for every array, releases in reverse order, inputs
 * with JNI_ABORT and the output with 0, no JNI call inside a critical section, GetDirectBufferAddress before any pin.
 * Difference that a GPU forces: a status comes back (0 = ok, negative = SKAINET_CUDA_ERR_*), the Kotlin side turns
 * it into IllegalArgumentException / IllegalStateException; and weights are uploaded once (uploadWeight -> handle)
 * so that a decode call carries only its activation row across PCIe.
 */
#include <jni.h>
#include <stddef.h>
#include <stdint.h>

#include "skainet_cuda.h"
#include "skainet_cuda_llama.h"

#define JNI_FN(name) Java_sk_ainet_exec_kernel_cuda_CudaKernels_##name

JNIEXPORT jstring JNICALL JNI_FN(lastError)(JNIEnv* env, jobject thiz) {
    (void) thiz;
    return (*env)->NewStringUTF(env, skainet_cuda_last_error());
}

JNIEXPORT jint JNICALL JNI_FN(deviceCount)(JNIEnv* env, jobject thiz) {
    (void) env; (void) thiz;
    return skainet_cuda_device_count();
}

JNIEXPORT jint JNICALL JNI_FN(deviceStatus)(JNIEnv* env, jobject thiz) {
    (void) env; (void) thiz;
    return skainet_cuda_device_status();
}

/* Availability probe: out[i] = 2 * in[i] on the GPU (JniKernelProvider.kt:36-45 calls the CPU twin of this). */
JNIEXPORT jint JNICALL JNI_FN(smoke)(JNIEnv* env, jobject thiz, jfloatArray input, jfloatArray output, jint length) {
    (void) thiz;
    jint st = SKAINET_CUDA_ERR_INVALID;
    jfloat* in = (*env)->GetPrimitiveArrayCritical(env, input, NULL);
    jfloat* out = in ? (*env)->GetPrimitiveArrayCritical(env, output, NULL) : NULL;
    if (out) st = skainet_cuda_smoke_double(in, out, length);
    if (out) (*env)->ReleasePrimitiveArrayCritical(env, output, out, 0);
    if (in) (*env)->ReleasePrimitiveArrayCritical(env, input, in, JNI_ABORT);
    return st;
}

/* ---- drop-in matvec twins: the whole weight crosses per call (what the SPI's ByteArray form implies) ---- */
#define SKAINET_JNI_MATMUL_BODY(CALL)                                              \
    jint st = SKAINET_CUDA_ERR_INVALID;                                            \
    jfloat* in = (*env)->GetPrimitiveArrayCritical(env, input, NULL);              \
    jbyte* w = in ? (*env)->GetPrimitiveArrayCritical(env, weight, NULL) : NULL;   \
    jfloat* out = w ? (*env)->GetPrimitiveArrayCritical(env, output, NULL) : NULL; \
    if (out) st = CALL;                                                            \
    if (out) (*env)->ReleasePrimitiveArrayCritical(env, output, out, 0);           \
    if (w) (*env)->ReleasePrimitiveArrayCritical(env, weight, w, JNI_ABORT);       \
    if (in) (*env)->ReleasePrimitiveArrayCritical(env, input, in, JNI_ABORT);      \
    return st;

#define SKAINET_JNI_MATMUL(jname, cname)                                                                     \
    JNIEXPORT jint JNICALL JNI_FN(jname)(JNIEnv* env, jobject thiz, jfloatArray input, jint inputOffset,     \
        jbyteArray weight, jint weightByteOffset, jint inputDim, jint outputDim, jfloatArray output, jint outputOffset) { \
        (void) thiz;                                                                                         \
        SKAINET_JNI_MATMUL_BODY(cname(in, inputOffset, (const uint8_t*) w, weightByteOffset, inputDim, outputDim, out, outputOffset)) \
    }

SKAINET_JNI_MATMUL(q4kMatmul, skainet_cuda_q4k_matmul)
SKAINET_JNI_MATMUL(q4kMatmulRm, skainet_cuda_q4k_matmul_rm)
SKAINET_JNI_MATMUL(q80Matmul, skainet_cuda_q8_0_matmul)
SKAINET_JNI_MATMUL(q80MatmulRm, skainet_cuda_q8_0_matmul_rm)
SKAINET_JNI_MATMUL(q6kMatmul, skainet_cuda_q6k_matmul)
SKAINET_JNI_MATMUL(q6kMatmulRm, skainet_cuda_q6k_matmul_rm)
SKAINET_JNI_MATMUL(q5kMatmul, skainet_cuda_q5k_matmul)
SKAINET_JNI_MATMUL(q5kMatmulRm, skainet_cuda_q5k_matmul_rm)

/* ---- resident weights: upload once, multiply many times ---- */
/* weight as a heap ByteArray; order 0 = row-major (GGUF file order), 1 = input-major ("feed order"). Returns the handle, or 0. */
JNIEXPORT jlong JNICALL JNI_FN(uploadWeight)(JNIEnv* env, jobject thiz, jbyteArray weight, jint byteOffset, jlong nbytes,
                                             jint encoding, jint rows, jint cols, jint order) {
    (void) thiz;
    skainet_weight_t h = 0;
    jbyte* w = (*env)->GetPrimitiveArrayCritical(env, weight, NULL);
    if (w) {
        if (skainet_cuda_weight_upload((const uint8_t*) w + byteOffset, nbytes, encoding, rows, cols, order, &h) != SKAINET_CUDA_OK) h = 0;
        (*env)->ReleasePrimitiveArrayCritical(env, weight, w, JNI_ABORT);
    }
    return (jlong) h;
}
/* weight as a direct (or mapped) ByteBuffer: the address is taken before anything is pinned (skainet_jni.c:146-167) */
JNIEXPORT jlong JNICALL JNI_FN(uploadWeightDirect)(JNIEnv* env, jobject thiz, jobject weight, jlong byteOffset, jlong nbytes,
                                                   jint encoding, jint rows, jint cols, jint order) {
    (void) thiz;
    skainet_weight_t h = 0;
    const uint8_t* w = (const uint8_t*) (*env)->GetDirectBufferAddress(env, weight);
    if (w && skainet_cuda_weight_upload(w + byteOffset, nbytes, encoding, rows, cols, order, &h) != SKAINET_CUDA_OK) h = 0;
    return (jlong) h;
}
JNIEXPORT jint JNICALL JNI_FN(freeWeight)(JNIEnv* env, jobject thiz, jlong handle) {
    (void) env; (void) thiz;
    return skainet_cuda_weight_free((skainet_weight_t) handle);
}

/* y[m, rows] = x[m, cols] . W^T for a resident weight; activation and output are heap FloatArrays (m rows from / to the
 * given element offsets). The activation is copied to a device buffer, the critical pins are released, the kernel runs,
 * and only then is the output pinned: no pin is held across the launch. */
JNIEXPORT jint JNICALL JNI_FN(matmulResident)(JNIEnv* env, jobject thiz, jlong handle, jfloatArray input, jint inputOffset, jint m,
                                              jint cols, jint rows, jfloatArray output, jint outputOffset) {
    (void) thiz;
    void *dx = NULL, *dy = NULL;
    const int64_t xb = (int64_t) m * cols * 4, yb = (int64_t) m * rows * 4;
    jint st = skainet_cuda_malloc(&dx, xb);
    if (st == SKAINET_CUDA_OK) st = skainet_cuda_malloc(&dy, yb);
    if (st == SKAINET_CUDA_OK) {
        jfloat* in = (*env)->GetPrimitiveArrayCritical(env, input, NULL);
        if (in) {
            st = skainet_cuda_memcpy_h2d(dx, in + inputOffset, xb, NULL);
            if (st == SKAINET_CUDA_OK) st = skainet_cuda_stream_sync(NULL);      /* the pin ends with the copy */
            (*env)->ReleasePrimitiveArrayCritical(env, input, in, JNI_ABORT);
        } else st = SKAINET_CUDA_ERR_INVALID;
    }
    if (st == SKAINET_CUDA_OK) st = skainet_cuda_matmul_dev((skainet_weight_t) handle, (const float*) dx, m, (float*) dy, SKAINET_ACT_NATIVE, NULL);
    if (st == SKAINET_CUDA_OK) {
        jfloat* out = (*env)->GetPrimitiveArrayCritical(env, output, NULL);
        if (out) {
            st = skainet_cuda_memcpy_d2h(out + outputOffset, dy, yb, NULL);      /* synchronises */
            (*env)->ReleasePrimitiveArrayCritical(env, output, out, 0);
        } else st = SKAINET_CUDA_ERR_INVALID;
    }
    skainet_cuda_free(dx);
    skainet_cuda_free(dy);
    return st;
}

/* ---- fused fp32 kernels (Fp32FusedKernels.kt:46-52,75-84) ---- */
JNIEXPORT jint JNICALL JNI_FN(rmsNorm)(JNIEnv* env, jobject thiz, jfloatArray input, jint inputOffset, jfloatArray gamma,
                                       jfloatArray out, jint outOffset, jint rows, jint cols, jfloat eps) {
    (void) thiz;
    jint st = SKAINET_CUDA_ERR_INVALID;
    jfloat* in = (*env)->GetPrimitiveArrayCritical(env, input, NULL);
    jfloat* g = (in && gamma) ? (*env)->GetPrimitiveArrayCritical(env, gamma, NULL) : NULL;
    jfloat* o = (in && (g || !gamma)) ? (*env)->GetPrimitiveArrayCritical(env, out, NULL) : NULL;
    if (o) st = skainet_cuda_f32_rms_norm(in + inputOffset, g, o + outOffset, rows, cols, eps);
    if (o) (*env)->ReleasePrimitiveArrayCritical(env, out, o, 0);
    if (g) (*env)->ReleasePrimitiveArrayCritical(env, gamma, g, JNI_ABORT);
    if (in) (*env)->ReleasePrimitiveArrayCritical(env, input, in, JNI_ABORT);
    return st;
}

JNIEXPORT jint JNICALL JNI_FN(sdpa)(JNIEnv* env, jobject thiz, jfloatArray query, jfloatArray key, jfloatArray value, jfloatArray out,
                                    jint batch, jint heads, jint kvHeads, jint seqQ, jint seqKV, jint headDim, jfloat scale,
                                    jboolean causal, jint window, jint rightContext, jintArray keyLengths, jfloatArray mask,
                                    jint maskB, jint maskH, jint maskQ, jint maskK) {
    (void) thiz;
    jint st = SKAINET_CUDA_ERR_INVALID;
    jfloat* q = (*env)->GetPrimitiveArrayCritical(env, query, NULL);
    jfloat* k = q ? (*env)->GetPrimitiveArrayCritical(env, key, NULL) : NULL;
    jfloat* v = k ? (*env)->GetPrimitiveArrayCritical(env, value, NULL) : NULL;
    jint* len = (v && keyLengths) ? (*env)->GetPrimitiveArrayCritical(env, keyLengths, NULL) : NULL;
    jfloat* mk = (v && mask) ? (*env)->GetPrimitiveArrayCritical(env, mask, NULL) : NULL;
    const int ok = v && (len || !keyLengths) && (mk || !mask);
    jfloat* o = ok ? (*env)->GetPrimitiveArrayCritical(env, out, NULL) : NULL;
    if (o) st = skainet_cuda_f32_sdpa(q, k, v, o, batch, heads, kvHeads, seqQ, seqKV, headDim, scale, causal ? 1 : 0, window, rightContext,
                                      (const int32_t*) len, mk, maskB, maskH, maskQ, maskK);
    if (o) (*env)->ReleasePrimitiveArrayCritical(env, out, o, 0);
    if (mk) (*env)->ReleasePrimitiveArrayCritical(env, mask, mk, JNI_ABORT);
    if (len) (*env)->ReleasePrimitiveArrayCritical(env, keyLengths, len, JNI_ABORT);
    if (v) (*env)->ReleasePrimitiveArrayCritical(env, value, v, JNI_ABORT);
    if (k) (*env)->ReleasePrimitiveArrayCritical(env, key, k, JNI_ABORT);
    if (q) (*env)->ReleasePrimitiveArrayCritical(env, query, q, JNI_ABORT);
    return st;
}

/* ---- KV-cache store (KvCacheStore.kt:125-157) ---- */
JNIEXPORT jlong JNICALL JNI_FN(kvCreate)(JNIEnv* env, jobject thiz, jint layers, jint heads, jint headDim, jint maxSeqLen, jboolean slidingWindow) {
    (void) env; (void) thiz;
    skainet_kv_t h = 0;
    if (skainet_cuda_kv_create(layers, heads, headDim, maxSeqLen, slidingWindow ? 1 : 0, &h) != SKAINET_CUDA_OK) h = 0;
    return (jlong) h;
}
/* TurboQuantKvCacheStore.kt:62-199: residual bits 0 = PolarOnly */
JNIEXPORT jlong JNICALL JNI_FN(kvCreateTurboquant)(JNIEnv* env, jobject thiz, jint layers, jint heads, jint headDim, jint maxSeqLen, jint keyBits,
                                                   jint keyResidualBits, jint valueBits, jint valueResidualBits) {
    (void) env; (void) thiz;
    skainet_kv_t h = 0;
    if (skainet_cuda_kv_create_turboquant(layers, heads, headDim, maxSeqLen, keyBits, keyResidualBits, valueBits, valueResidualBits, &h) != SKAINET_CUDA_OK) h = 0;
    return (jlong) h;
}
JNIEXPORT jint JNICALL JNI_FN(kvFree)(JNIEnv* env, jobject thiz, jlong kv) { (void) env; (void) thiz; return skainet_cuda_kv_free((skainet_kv_t) kv); }
JNIEXPORT jint JNICALL JNI_FN(kvEvict)(JNIEnv* env, jobject thiz, jlong kv, jint fromPos) { (void) env; (void) thiz; return skainet_cuda_kv_evict((skainet_kv_t) kv, fromPos); }
JNIEXPORT jint JNICALL JNI_FN(kvClear)(JNIEnv* env, jobject thiz, jlong kv) { (void) env; (void) thiz; return skainet_cuda_kv_clear((skainet_kv_t) kv); }
JNIEXPORT jint JNICALL JNI_FN(kvAppend)(JNIEnv* env, jobject thiz, jlong kv, jint layer, jfloatArray key, jfloatArray value) {
    (void) thiz;
    jint st = SKAINET_CUDA_ERR_INVALID;
    jfloat* k = (*env)->GetPrimitiveArrayCritical(env, key, NULL);
    jfloat* v = k ? (*env)->GetPrimitiveArrayCritical(env, value, NULL) : NULL;
    if (v) st = skainet_cuda_kv_append((skainet_kv_t) kv, layer, k, v);
    if (v) (*env)->ReleasePrimitiveArrayCritical(env, value, v, JNI_ABORT);
    if (k) (*env)->ReleasePrimitiveArrayCritical(env, key, k, JNI_ABORT);
    return st;
}
JNIEXPORT jint JNICALL JNI_FN(kvRead)(JNIEnv* env, jobject thiz, jlong kv, jint layer, jint which, jint startPos, jint endPos, jfloatArray out) {
    (void) thiz;
    jint st = SKAINET_CUDA_ERR_INVALID;
    jfloat* o = (*env)->GetPrimitiveArrayCritical(env, out, NULL);
    if (o) {
        st = skainet_cuda_kv_read((skainet_kv_t) kv, layer, which, startPos, endPos, o);
        (*env)->ReleasePrimitiveArrayCritical(env, out, o, 0);
    }
    return st;
}
JNIEXPORT jint JNICALL JNI_FN(kvInfo)(JNIEnv* env, jobject thiz, jlong kv, jlongArray out8) {
    (void) thiz;
    jint st = SKAINET_CUDA_ERR_INVALID;
    jlong* o = (*env)->GetPrimitiveArrayCritical(env, out8, NULL);
    if (o) {
        st = skainet_cuda_kv_info((skainet_kv_t) kv, (int64_t*) o);
        (*env)->ReleasePrimitiveArrayCritical(env, out8, o, 0);
    }
    return st;
}
