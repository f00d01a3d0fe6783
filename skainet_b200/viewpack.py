"""Host-side mirror of the view-kernel pack a CUDA backend registers into the reference's KernelDispatch: `x . W^T` over a
packed weight view, keyed like the CPU packs' kernels (dense contiguous FP32 activation x Format(FP32, encoding) weight in
BLOCKED_ROW_MAJOR or BLOCKED_INPUT_MAJOR order; skainet-backends/skainet-backend-native-cpu/src/jvmMain/kotlin/sk/ainet/
exec/kernel/FfmRowMajorKernels.kt:42-170), with the part that makes the SPI path usable on a GPU: the weight of a view is
uploaded to HBM on FIRST use and found again by the IDENTITY of its storage (the pattern of WasmRowMajorMatmulKernel's
weightHandle, skainet-backends/skainet-backend-wasm-simd/src/wasmJsMain/kotlin/sk/ainet/exec/wasm/
WasmRowMajorMatmulKernel.kt:27-73), so a decode call moves only its activation rows over PCIe. Entries die with their
storage and the device copy is freed then. This is the tested twin of skainet_b200/jvm/.../CudaViewKernelPack.kt.

No CPU fallback: a view this kernel cannot take (strided activation, wrong block order, wrong shapes) is refused with an
exception naming the reason."""
from __future__ import annotations

import threading
import weakref
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from . import _lib as L

ROW_MAJOR, INPUT_MAJOR = "BLOCKED_ROW_MAJOR", "BLOCKED_INPUT_MAJOR"
ENCODINGS = ("Q4_K", "Q8_0", "Q6_K", "Q5_K")       # the encodings FfmRowMajorKernelPack serves that the library has kernels for


@dataclass(eq=False)
class PackedWeightView:
    """A [n, k] weight as packed blocks: `storage` holds the bytes in `order` (file order or feed order)."""
    storage: np.ndarray
    shape: Tuple[int, int]
    encoding: str
    order: str = ROW_MAJOR
    byte_offset: int = 0


class DeviceBackend:
    """What the kernel needs from the device: upload once, multiply many times, free. The default goes through the C ABI
    (skainet_cuda_weight_upload / skainet_cuda_matmul_dev / skainet_cuda_weight_free); tests inject a recording fake."""

    def upload(self, packed: np.ndarray, encoding: str, n: int, k: int, order: str):
        from .device import Weight
        return Weight.upload(packed, encoding, n, k, L.ORDER_ROW_MAJOR if order == ROW_MAJOR else L.ORDER_INPUT_MAJOR)

    def matmul(self, handle, x: np.ndarray, out: np.ndarray) -> None:
        from .device import matmul_host
        out[...] = matmul_host(handle, x).reshape(out.shape)

    def free(self, handle) -> None:
        handle.free()


def key_for(encoding: str, order: str) -> Tuple[str, str, str, str]:
    """op, activation format, weight format, weight block order: the fields of the reference's KernelKey for this kernel."""
    return ("matmul", "FP32", f"FP32/{encoding}", order)


class CudaPackedMatmulKernel:
    """One (encoding, block order) of the pack. `run([activation, weight_view], out)`."""

    _lock = threading.Lock()
    _resident: Dict[int, object] = {}          # id(storage) -> device handle; the finalizer of the storage removes the entry

    def __init__(self, encoding: str, order: str, backend: Optional[DeviceBackend] = None):
        if encoding not in ENCODINGS:
            raise ValueError(f"encoding {encoding} has no GPU view kernel")
        self.encoding, self.order = encoding, order
        self.key = key_for(encoding, order)
        self.name = f"cuda-sm100-{encoding.lower()}-{'rm' if order == ROW_MAJOR else 'im'}"
        self.backend = backend or DeviceBackend()

    def run(self, inputs: List[object], out: np.ndarray) -> None:
        if len(inputs) != 2:
            raise ValueError("matmul takes two operands")
        a, w = inputs
        if not isinstance(a, np.ndarray) or a.dtype != np.float32 or a.ndim != 2:
            raise TypeError(f"{self.name}: activation must be a 2-d float32 array")
        if not isinstance(w, PackedWeightView):
            raise TypeError(f"{self.name}: weight must be a packed view")
        rows, k = a.shape
        n, wk = w.shape
        if wk != k:
            raise ValueError(f"inner dimensions disagree: [{rows}, {k}] x [{n}, {wk}]")
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError(f"{self.name} takes a contiguous activation")
        if not isinstance(out, np.ndarray) or out.dtype != np.float32 or out.shape != (rows, n) or not out.flags["C_CONTIGUOUS"]:
            raise ValueError(f"{self.name}: output must be a contiguous float32 [{rows}, {n}] array")
        self.backend.matmul(self._resident_handle(w, n, k), a, out)

    def _resident_handle(self, w: PackedWeightView, n: int, k: int):
        """The device copy of the view's bytes: uploaded once per storage object, in the order the view declares."""
        if w.encoding != self.encoding or w.order != self.order:
            raise ValueError(f"{self.name}: weight is {w.encoding} in {w.order}, which does not match the key")
        storage = w.storage
        cache, backend = CudaPackedMatmulKernel._resident, self.backend
        with CudaPackedMatmulKernel._lock:
            hit = cache.get(id(storage))
            if hit is not None:
                return hit
            be, bb = L.BLOCK_ELEMS[self.encoding], L.BLOCK_BYTES[self.encoding]
            if k % be != 0:
                raise ValueError(f"{self.name}: inputDim must be a multiple of {be}; got {k}")
            nbytes = n * (k // be) * bb
            flat = storage.reshape(-1).view(np.uint8)
            if flat.size - w.byte_offset < nbytes:
                raise IndexError(f"{self.name}: the view's storage holds {flat.size - w.byte_offset} bytes, the weight needs {nbytes}")
            handle = backend.upload(flat[w.byte_offset:w.byte_offset + nbytes], self.encoding, n, k, self.order)
            key = id(storage)
            cache[key] = handle

            def release(key=key, handle=handle, backend=backend, cache=cache, lock=CudaPackedMatmulKernel._lock):
                with lock:
                    cache.pop(key, None)
                backend.free(handle)

            weakref.finalize(storage, release)          # the device copy goes when the storage object does
            return handle


class KernelDispatch:
    """The slice of the reference's registry the pack uses: exact-match lookup, a later registration replaces an earlier one
    (skainet-backends/skainet-backend-api/src/commonMain/kotlin/sk/ainet/backend/api/kernel/KernelDispatch.kt)."""

    def __init__(self) -> None:
        self._kernels: Dict[Tuple[str, str, str, str], CudaPackedMatmulKernel] = {}

    def register(self, kernel) -> None:
        self._kernels[kernel.key] = kernel

    def lookup(self, key):
        return self._kernels.get(key)

    def __len__(self) -> int:
        return len(self._kernels)


class CudaViewKernelPack:
    """Registers the GPU view kernels: every encoding of ENCODINGS in both block orders. Idempotent, and a no-op while
    the provider is unavailable (the ViewKernelPack.install contract)."""

    name = "cuda-sm100-packed"

    def __init__(self, available: Optional[Callable[[], bool]] = None, backend: Optional[DeviceBackend] = None):
        if available is None:
            from .provider import CudaKernelProvider
            available = CudaKernelProvider().isAvailable
        self._available, self._backend, self._installed = available, backend, False

    def install(self, dispatch: KernelDispatch) -> None:
        if self._installed or not self._available():
            return
        for enc in ENCODINGS:
            for order in (ROW_MAJOR, INPUT_MAJOR):
                dispatch.register(CudaPackedMatmulKernel(enc, order, self._backend))
        self._installed = True
