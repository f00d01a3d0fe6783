package sk.ainet.exec.kernel.cuda

/**
 * JNI surface over `libskainet_cuda.so` through the shim `libskainet_cuda_jni.so`
 * (native/skainet_cuda_jni.c). One `external fun` per C entry point; names carry no underscore
 * because JNI mangles `_` to `_1` in native symbol names (the rule of
 * skainet-backend-jni-cpu's `JniKernels`).
 *
 * UNVERIFIED SOURCE: written to the reference's JNI pattern; no JDK / Kotlin compiler exists where
 * the native library is built and tested. The C ABI behind every call is tested from Python.
 *
 * Every compute call returns a status: 0 = ok, negative = `SKAINET_CUDA_ERR_*`
 * (-1 invalid argument, -2 CUDA error, -3 no device, -4 out of memory, -5 bad handle, -6 a bounded
 * device wait gave up, -7 collective library). [check] turns it into the exception the SPI
 * contracts name.
 */
public object CudaKernels {

    /** Loaded eagerly in object init, so a direct call to any `external fun` finds the library. */
    public val isLoaded: Boolean = runCatching {
        System.loadLibrary("skainet_cuda")        // the kernels; resolved first so the shim's imports bind
        System.loadLibrary("skainet_cuda_jni")
        true
    }.getOrDefault(false)

    public external fun lastError(): String
    public external fun deviceCount(): Int
    public external fun deviceStatus(): Int
    public external fun smoke(input: FloatArray, output: FloatArray, length: Int): Int

    // drop-in matvec twins: the weight crosses on every call
    public external fun q4kMatmul(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q4kMatmulRm(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q80Matmul(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q80MatmulRm(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q6kMatmul(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q6kMatmulRm(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q5kMatmul(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int
    public external fun q5kMatmulRm(input: FloatArray, inputOffset: Int, weight: ByteArray, weightByteOffset: Int, inputDim: Int, outputDim: Int, output: FloatArray, outputOffset: Int): Int

    // resident weights: upload once (handle, or 0 on failure), multiply many times
    public external fun uploadWeight(weight: ByteArray, byteOffset: Int, nbytes: Long, encoding: Int, rows: Int, cols: Int, order: Int): Long
    public external fun uploadWeightDirect(weight: java.nio.ByteBuffer, byteOffset: Long, nbytes: Long, encoding: Int, rows: Int, cols: Int, order: Int): Long
    public external fun freeWeight(handle: Long): Int
    public external fun matmulResident(handle: Long, input: FloatArray, inputOffset: Int, m: Int, cols: Int, rows: Int, output: FloatArray, outputOffset: Int): Int

    // fused fp32 kernels
    public external fun rmsNorm(input: FloatArray, inputOffset: Int, gamma: FloatArray?, out: FloatArray, outOffset: Int, rows: Int, cols: Int, eps: Float): Int
    public external fun sdpa(
        query: FloatArray, key: FloatArray, value: FloatArray, out: FloatArray,
        batch: Int, heads: Int, kvHeads: Int, seqQ: Int, seqKV: Int, headDim: Int, scale: Float, causal: Boolean, window: Int, rightContext: Int,
        keyLengths: IntArray?, mask: FloatArray?, maskB: Int, maskH: Int, maskQ: Int, maskK: Int,
    ): Int

    // KV-cache store
    public external fun kvCreate(layers: Int, heads: Int, headDim: Int, maxSeqLen: Int, slidingWindow: Boolean): Long
    public external fun kvCreateTurboquant(layers: Int, heads: Int, headDim: Int, maxSeqLen: Int, keyBits: Int, keyResidualBits: Int,
                                           valueBits: Int, valueResidualBits: Int): Long
    public external fun kvFree(kv: Long): Int
    public external fun kvAppend(kv: Long, layer: Int, key: FloatArray, value: FloatArray): Int
    public external fun kvRead(kv: Long, layer: Int, which: Int, startPos: Int, endPos: Int, out: FloatArray): Int
    public external fun kvEvict(kv: Long, fromPos: Int): Int
    public external fun kvClear(kv: Long): Int
    public external fun kvInfo(kv: Long, out8: LongArray): Int

    public const val ENC_Q8_0: Int = 8
    public const val ENC_Q4_K: Int = 12
    public const val ENC_Q5_K: Int = 13
    public const val ENC_Q6_K: Int = 14
    public const val ORDER_ROW_MAJOR: Int = 0
    public const val ORDER_INPUT_MAJOR: Int = 1

    /** 0 passes; -1 is the SPI's `IllegalArgumentException`; anything else is a failed GPU call (there is no CPU fallback). */
    public fun check(status: Int) {
        when (status) {
            0 -> Unit
            -1 -> throw IllegalArgumentException(lastError())
            -4 -> throw OutOfMemoryError(lastError())
            else -> throw IllegalStateException("skainet-backend-cuda [$status]: ${lastError()}")
        }
    }
}
