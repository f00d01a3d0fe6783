package sk.ainet.exec.kernel.cuda

import sk.ainet.backend.api.kernel.Fp32AttentionKernel
import sk.ainet.backend.api.kernel.Fp32MatmulKernel
import sk.ainet.backend.api.kernel.Fp32NormKernel
import sk.ainet.backend.api.kernel.KernelProvider
import sk.ainet.backend.api.kernel.Q4KMatmulKernel
import sk.ainet.backend.api.kernel.Q5KMatmulKernel
import sk.ainet.backend.api.kernel.Q6KMatmulKernel
import sk.ainet.backend.api.kernel.Q8_0MatmulKernel

/**
 * Priority-200 [KernelProvider] over the B200 kernels of `libskainet_cuda.so`: above the FFM / JNI CPU
 * providers (100), so the registry prefers it wherever a GPU answers.
 *
 * UNVERIFIED SOURCE (no Kotlin toolchain where the library is built); the Python mirror
 * `skainet_b200/provider.py` implements the same accessors over the same C ABI and is what the tests run.
 *
 * Availability is probed once, like `JniKernelProvider`: the libraries must have loaded, a device must be
 * present and the smoke kernel must round-trip. When it does not, [isAvailable] is false and the registry
 * cascades to the CPU providers — but once selected, a kernel of this provider never falls back to the
 * CPU: a failed GPU call throws.
 *
 * The matvec accessors here serve the legacy SPI whose `weight: ByteArray` crosses on every call
 * (correct, slow: PCIe carries the weight each time). The fast path is [CudaViewKernelPack], which keeps
 * each weight resident on the device, keyed by its storage identity.
 */
public object CudaKernelProvider : KernelProvider {

    override val name: String = "cuda-sm100"

    override val priority: Int = 200

    private val available: Boolean by lazy {
        if (!CudaKernels.isLoaded || CudaKernels.deviceCount() <= 0) return@lazy false
        runCatching {
            val input = floatArrayOf(1.0f, 2.5f, -3.0f)
            val output = FloatArray(3)
            CudaKernels.smoke(input, output, 3) == 0 && output[0] == 2.0f && output[1] == 5.0f && output[2] == -6.0f
        }.getOrDefault(false)
    }

    override fun isAvailable(): Boolean = available

    override fun matmulFp32(): Fp32MatmulKernel? = null          // dense fp32 GEMM is not on this backend's path

    override fun matmulQ4K(): Q4KMatmulKernel? = if (available) CudaQ4KMatmul else null

    override fun matmulQ8_0(): Q8_0MatmulKernel? = if (available) CudaQ80Matmul else null

    override fun matmulQ6K(): Q6KMatmulKernel? = if (available) CudaQ6KMatmul else null

    override fun matmulQ5K(): Q5KMatmulKernel? = if (available) CudaQ5KMatmul else null

    override fun normFp32(): Fp32NormKernel? = if (available) CudaNorm else null

    override fun attentionFp32(): Fp32AttentionKernel? = if (available) CudaAttention else null

    private object CudaQ4KMatmul : Q4KMatmulKernel {
        override fun matmul(
            input: FloatArray, inputOffset: Int,
            weight: ByteArray, weightByteOffset: Int,
            inputDim: Int, outputDim: Int,
            output: FloatArray, outputOffset: Int,
        ): Unit = CudaKernels.check(CudaKernels.q4kMatmul(input, inputOffset, weight, weightByteOffset, inputDim, outputDim, output, outputOffset))
    }

    private object CudaQ80Matmul : Q8_0MatmulKernel {
        override fun matmul(
            input: FloatArray, inputOffset: Int,
            weight: ByteArray, weightByteOffset: Int,
            inputDim: Int, outputDim: Int,
            output: FloatArray, outputOffset: Int,
        ): Unit = CudaKernels.check(CudaKernels.q80Matmul(input, inputOffset, weight, weightByteOffset, inputDim, outputDim, output, outputOffset))
    }

    private object CudaQ6KMatmul : Q6KMatmulKernel {
        override fun matmul(
            input: FloatArray, inputOffset: Int,
            weight: ByteArray, weightByteOffset: Int,
            inputDim: Int, outputDim: Int,
            output: FloatArray, outputOffset: Int,
        ): Unit = CudaKernels.check(CudaKernels.q6kMatmul(input, inputOffset, weight, weightByteOffset, inputDim, outputDim, output, outputOffset))
    }

    private object CudaQ5KMatmul : Q5KMatmulKernel {
        override fun matmul(
            input: FloatArray, inputOffset: Int,
            weight: ByteArray, weightByteOffset: Int,
            inputDim: Int, outputDim: Int,
            output: FloatArray, outputOffset: Int,
        ): Unit = CudaKernels.check(CudaKernels.q5kMatmul(input, inputOffset, weight, weightByteOffset, inputDim, outputDim, output, outputOffset))
    }

    private object CudaNorm : Fp32NormKernel {
        override fun layerNorm(
            input: FloatArray, inputOffset: Int,
            gamma: FloatArray?, beta: FloatArray?,
            out: FloatArray, outOffset: Int,
            rows: Int, cols: Int,
            eps: Float,
        ): Unit = throw UnsupportedOperationException("skainet-backend-cuda serves rmsNorm only (the Llama path); layerNorm stays with the CPU provider")

        override fun rmsNorm(
            input: FloatArray, inputOffset: Int,
            gamma: FloatArray?,
            out: FloatArray, outOffset: Int,
            rows: Int, cols: Int,
            eps: Float,
        ): Unit = CudaKernels.check(CudaKernels.rmsNorm(input, inputOffset, gamma, out, outOffset, rows, cols, eps))
    }

    private object CudaAttention : Fp32AttentionKernel {
        override fun sdpa(
            query: FloatArray, key: FloatArray, value: FloatArray, out: FloatArray,
            batch: Int, heads: Int, kvHeads: Int,
            seqQ: Int, seqKV: Int, headDim: Int,
            scale: Float, causal: Boolean, window: Int, rightContext: Int,
            keyLengths: IntArray?,
            mask: FloatArray?, maskDims: IntArray?,
        ) {
            val md = maskDims ?: intArrayOf(0, 0, 0, 0)
            require(mask == null || md.size == 4) { "maskDims must be [batch, heads, seqQ, seqKV] broadcast sizes" }
            CudaKernels.check(
                CudaKernels.sdpa(query, key, value, out, batch, heads, kvHeads, seqQ, seqKV, headDim, scale, causal, window, rightContext,
                    keyLengths, mask, md[0], md[1], md[2], md[3]),
            )
        }
    }
}

/** Public no-arg class for `META-INF/services/sk.ainet.backend.api.kernel.KernelProvider` (ServiceLoader needs a constructor). */
public class CudaKernelProviderFactory : KernelProvider by CudaKernelProvider
