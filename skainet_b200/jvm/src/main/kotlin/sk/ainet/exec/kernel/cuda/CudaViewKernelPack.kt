package sk.ainet.exec.kernel.cuda

import sk.ainet.backend.api.kernel.KernelDispatch
import sk.ainet.backend.api.kernel.KernelKey
import sk.ainet.backend.api.kernel.LayoutClass
import sk.ainet.backend.api.kernel.OperandKey
import sk.ainet.backend.api.kernel.ViewKernel
import sk.ainet.backend.api.kernel.ViewKernelPack
import sk.ainet.lang.memory.BlockOrder
import sk.ainet.lang.memory.Format
import sk.ainet.lang.memory.Storage
import sk.ainet.lang.memory.TensorView
import sk.ainet.lang.memory.trace.NoopTraceSink
import sk.ainet.lang.memory.trace.TraceEvent
import sk.ainet.lang.memory.trace.TraceSink
import sk.ainet.lang.tensor.storage.TensorEncoding
import sk.ainet.lang.types.FP32
import java.util.Collections
import java.util.WeakHashMap

/**
 * `x · Wᵀ` over a packed weight on the GPU, registered under the same view keys the CPU packs serve
 * (dense contiguous FP32 activation × `Format(FP32, encoding)` weight in `BLOCKED_ROW_MAJOR` or
 * `BLOCKED_INPUT_MAJOR` order), after them, so this one wins the exact-match lookup
 * (`KernelDispatch.register`: later registration replaces).
 *
 * UNVERIFIED SOURCE (no Kotlin toolchain where the library is built). The resident-weight logic it
 * carries is the point: the weight of a view is uploaded to HBM on first use and found again by the
 * IDENTITY of its storage (the pattern of `WasmRowMajorMatmulKernel`'s `weightHandle` and of the CPU ops'
 * `prepackedWeights`), so a decode call moves only its activation rows across PCIe. Entries die with
 * their storage (weak keys); the handle is freed then.
 *
 * No CPU fallback: a view this kernel cannot take (strided activation, non-heap storage) is refused with
 * an exception naming the reason, where the CPU packs would trace `reference-fallback`.
 */
public class CudaPackedMatmulKernel internal constructor(
    private val encoding: TensorEncoding,
    private val encodingId: Int,
    private val order: LayoutClass,
) : ViewKernel {
    override val key: KernelKey = keyFor(encoding, order)
    override val name: String = "cuda-sm100-${encoding.name.lowercase()}-${if (order == LayoutClass.BLOCKED_ROW_MAJOR) "rm" else "im"}"

    override fun run(inputs: List<TensorView>, out: TensorView): Unit = run(inputs, out, NoopTraceSink)

    override fun run(inputs: List<TensorView>, out: TensorView, sink: TraceSink) {
        require(inputs.size == 2) { "matmul takes two operands" }
        val a = inputs[0]
        val w = inputs[1]
        val rows = a.shape[0]
        val k = a.shape[1]
        val n = w.shape[0]
        require(w.shape[1] == k) { "inner dimensions disagree: [$rows, $k] × [$n, ${w.shape[1]}]" }
        check(a.isContiguous) { "$name takes a contiguous activation" }
        val aHeap = a.storage as? Storage.Heap ?: error("$name: activation storage ${a.storage::class.simpleName}")
        val oHeap = out.storage as? Storage.Heap ?: error("$name: output storage ${out.storage::class.simpleName}")
        val activation = aHeap.floats ?: error("$name: activation is not a FloatArray")
        val output = oHeap.floats ?: error("$name: output is not a FloatArray")
        val handle = residentHandle(w, n, k)
        CudaKernels.check(
            CudaKernels.matmulResident(
                handle, activation, aHeap.arrayOffset + a.layout.offsetElements.toInt(), rows, k, n,
                output, oHeap.arrayOffset + out.layout.offsetElements.toInt(),
            ),
        )
        if (sink.isEnabled) sink.emit(TraceEvent.KernelRun(op = key.op, kernel = name, inputs = inputs.map { it.id }, output = out.id))
    }

    /** The device copy of [w]'s bytes: uploaded once per storage object, in the order the view declares. */
    private fun residentHandle(w: TensorView, n: Int, k: Int): Long {
        val storage = w.storage
        synchronized(resident) {
            resident[storage]?.let { return it.handle }
            val wantRowMajor = order == LayoutClass.BLOCKED_ROW_MAJOR
            check((w.layout.blockOrder == BlockOrder.ROW_MAJOR) == wantRowMajor) { "$name: weight block order ${w.layout.blockOrder} does not match the key" }
            val byteOffset = w.layout.offsetElements * w.layout.elementBytes
            val nbytes = storage.sizeBytes - byteOffset
            val orderId = if (wantRowMajor) CudaKernels.ORDER_ROW_MAJOR else CudaKernels.ORDER_INPUT_MAJOR
            val heap = storage as? Storage.Heap
            val bytes = heap?.bytes
            val handle = when {
                bytes != null -> CudaKernels.uploadWeight(bytes, heap.arrayOffset + byteOffset.toInt(), nbytes, encodingId, n, k, orderId)
                else -> {
                    val direct = storage.directBuffer() ?: error("$name: weight storage ${storage::class.simpleName} is neither a heap array nor a direct buffer")
                    CudaKernels.uploadWeightDirect(direct, byteOffset, nbytes, encodingId, n, k, orderId)
                }
            }
            check(handle != 0L) { "skainet-backend-cuda: weight upload failed: ${CudaKernels.lastError()}" }
            resident[storage] = Resident(handle)
            return handle
        }
    }

    /** Frees the device copy when the entry is collected with its storage. */
    private class Resident(val handle: Long) {
        @Suppress("unused")
        private val cleanable = cleaner.register(this, Release(handle))
    }

    private class Release(private val handle: Long) : Runnable {
        override fun run() { CudaKernels.freeWeight(handle) }
    }

    public companion object {
        private val cleaner: java.lang.ref.Cleaner = java.lang.ref.Cleaner.create()

        /** storage identity -> device weight; weak keys, so a weight's HBM goes when its tensor does. */
        private val resident: MutableMap<Storage, Resident> = Collections.synchronizedMap(WeakHashMap())

        public fun keyFor(encoding: TensorEncoding, order: LayoutClass): KernelKey = KernelKey(
            op = "matmul",
            operands = listOf(
                OperandKey.contiguous(Format.dense(FP32)),
                OperandKey(Format(FP32, encoding), order),
            ),
        )
    }
}

/**
 * Registers the GPU view kernels into [KernelDispatch]: Q4_K, Q8_0, Q6_K and Q5_K (the encodings `FfmRowMajorKernelPack`
 * serves that the library has kernels for), both block orders. Idempotent, and a
 * no-op when the provider is unavailable (`ViewKernelPack.install` contract).
 */
public object CudaViewKernelPack : ViewKernelPack {
    override val name: String = "cuda-sm100-packed"

    private var installed = false

    @Synchronized
    override fun install() {
        if (installed || !CudaKernelProvider.isAvailable()) return
        for ((encoding, id) in listOf(
            TensorEncoding.Q4_K to CudaKernels.ENC_Q4_K, TensorEncoding.Q8_0 to CudaKernels.ENC_Q8_0,
            TensorEncoding.Q6_K to CudaKernels.ENC_Q6_K, TensorEncoding.Q5_K to CudaKernels.ENC_Q5_K,
        )) {
            for (order in listOf(LayoutClass.BLOCKED_ROW_MAJOR, LayoutClass.BLOCKED_INPUT_MAJOR)) {
                KernelDispatch.register(CudaPackedMatmulKernel(encoding, id, order))
            }
        }
        installed = true
    }
}

/** Public no-arg class for `META-INF/services/sk.ainet.backend.api.kernel.ViewKernelPack`. */
public class CudaViewKernelPackFactory : ViewKernelPack by CudaViewKernelPack
