"""Host-side mirror of the reference's kernel SPI for the CUDA backend.

The reference's host language (Kotlin) has no toolchain here, so the classes a Kotlin
``CudaKernelProvider`` would hold are written in Python with the same names, argument order, and
error behaviour, each delegating 1:1 to the C ABI — exactly what the Kotlin classes would do through
JNI. ``FloatArray``/``ByteArray``/``IntArray`` are contiguous numpy arrays of float32/uint8/int32.

Mirrored interfaces (skainet-backends/skainet-backend-api/src/commonMain/kotlin/sk/ainet/backend/api/kernel/):
``KernelProvider`` (KernelProvider.kt:22-190), ``Q4KMatmulKernel`` (Q4KMatmulKernel.kt:43-73),
``Q8_0MatmulKernel`` (Q8_0MatmulKernel.kt:31-48), ``Fp32NormKernel`` / ``Fp32AttentionKernel``
(Fp32FusedKernels.kt:37-84). Row-major twins mirror ``FfmRowMajorMatmulKernel``
(skainet-backends/skainet-backend-native-cpu/src/jvmMain/kotlin/sk/ainet/exec/kernel/FfmRowMajorKernels.kt:52-105).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib as L


def _f32(a: np.ndarray, name: str) -> np.ndarray:
    if not (isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous):
        raise TypeError(f"{name} must be a C-contiguous float32 numpy array")
    return a


def _u8(a: np.ndarray, name: str) -> np.ndarray:
    if not (isinstance(a, np.ndarray) and a.dtype == np.uint8 and a.flags.c_contiguous):
        raise TypeError(f"{name} must be a C-contiguous uint8 numpy array")
    return a


def _fp(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(L.f32p)


class _PackedMatmulKernel:
    """``matmul(input, inputOffset, weight, weightByteOffset, inputDim, outputDim, output, outputOffset)``.

    Must not mutate its inputs and fully writes ``outputDim`` floats; ``inputDim`` not a multiple of the
    block size raises ``ValueError`` (the SPI's IllegalArgumentException)."""

    _enc = ""
    _entry = ""

    def __init__(self, row_major: bool = False):
        self.row_major = row_major

    def matmul(self, input: np.ndarray, inputOffset: int, weight: np.ndarray, weightByteOffset: int,
               inputDim: int, outputDim: int, output: np.ndarray, outputOffset: int) -> None:
        _f32(input, "input"); _u8(weight, "weight"); _f32(output, "output")
        be, bb = L.BLOCK_ELEMS[self._enc], L.BLOCK_BYTES[self._enc]
        if inputDim % be != 0:
            raise ValueError(f"{type(self).__name__}: inputDim must be a multiple of {be}; got {inputDim}")
        if inputDim > 0 and outputDim > 0:
            if input.size < inputOffset + inputDim or output.size < outputOffset + outputDim:
                raise IndexError("input/output array too small for the given offsets and dims")
            if weight.size < weightByteOffset + (inputDim // be) * outputDim * bb:
                raise IndexError("weight array too small for the given offset and dims")
        fn = getattr(L.lib(), self._entry + ("_rm" if self.row_major else ""))
        L.check(fn(_fp(input), inputOffset, weight.ctypes.data_as(L.u8p), weightByteOffset, inputDim, outputDim,
                   _fp(output), outputOffset))


class CudaQ4KMatmulKernel(_PackedMatmulKernel):
    """Q4_K matvec on the GPU; replaces NativeQ4KMatmulKernel
    (skainet-backends/skainet-backend-native-cpu/src/jvmMain/kotlin/sk/ainet/exec/kernel/NativeQ4KMatmulKernel.kt:42-85)."""
    _enc, _entry = "Q4_K", "skainet_cuda_q4k_matmul"


class CudaQ8_0MatmulKernel(_PackedMatmulKernel):
    _enc, _entry = "Q8_0", "skainet_cuda_q8_0_matmul"


class CudaQ6KMatmulKernel(_PackedMatmulKernel):
    """Q6_K matvec on the GPU (SPI Q6KMatmulKernel.kt; replaces the native kernel behind skainet_q6k_matmul / _rm,
    skainet-backends/skainet-backend-native-cpu/native/src/q6k_matmul.c:272-357)."""
    _enc, _entry = "Q6_K", "skainet_cuda_q6k_matmul"


class CudaQ5KMatmulKernel(_PackedMatmulKernel):
    """Q5_K matvec on the GPU (SPI Q5KMatmulKernel.kt; skainet_q5k_matmul / _rm, native/src/q5k_matmul.c)."""
    _enc, _entry = "Q5_K", "skainet_cuda_q5k_matmul"


class CudaFp32NormKernel:
    """``rmsNorm(input, inputOffset, gamma, out, outOffset, rows, cols, eps)`` — Fp32FusedKernels.kt:46-52."""

    def rmsNorm(self, input: np.ndarray, inputOffset: int, gamma: Optional[np.ndarray], out: np.ndarray,
                outOffset: int, rows: int, cols: int, eps: float) -> None:
        _f32(input, "input"); _f32(out, "out")
        if gamma is not None:
            _f32(gamma, "gamma")
        if rows <= 0 or cols <= 0:
            return
        src = input.reshape(-1)[inputOffset:inputOffset + rows * cols]
        dst = out.reshape(-1)[outOffset:outOffset + rows * cols]
        if src.size != rows * cols or dst.size != rows * cols:
            raise IndexError("input/out array too small for rows*cols at the given offset")
        L.check(L.lib().skainet_cuda_f32_rms_norm(_fp(src), _fp(gamma), _fp(dst), rows, cols, eps))

    def layerNorm(self, *args, **kwargs):
        raise NotImplementedError("layer_norm is outside the decode path this backend accelerates")


class CudaFp32AttentionKernel:
    """``sdpa(query, key, value, out, batch, heads, kvHeads, seqQ, seqKV, headDim, scale, causal, window,
    rightContext, keyLengths, mask, maskDims)`` — Fp32FusedKernels.kt:75-84."""

    def sdpa(self, query: np.ndarray, key: np.ndarray, value: np.ndarray, out: np.ndarray, batch: int, heads: int,
             kvHeads: int, seqQ: int, seqKV: int, headDim: int, scale: float, causal: bool, window: int,
             rightContext: int, keyLengths: Optional[np.ndarray], mask: Optional[np.ndarray],
             maskDims: Optional[Sequence[int]]) -> None:
        _f32(query, "query"); _f32(key, "key"); _f32(value, "value"); _f32(out, "out")
        lp = None
        if keyLengths is not None:
            if keyLengths.dtype != np.int32:
                raise TypeError("keyLengths must be int32")
            lp = keyLengths.ctypes.data_as(L.i32p)
        md = (0, 0, 0, 0)
        if mask is not None:
            _f32(mask, "mask")
            md = tuple(int(x) for x in (maskDims if maskDims is not None else mask.shape))
            md = (1,) * (4 - len(md)) + md
        L.check(L.lib().skainet_cuda_f32_sdpa(_fp(query), _fp(key), _fp(value), _fp(out), batch, heads, kvHeads, seqQ, seqKV,
                                              headDim, scale, int(bool(causal)), window, rightContext, lp, _fp(mask), *md))


class CudaKernelProvider:
    """The provider a ServiceLoader entry would expose: highest priority, available only when the
    GPU answers the smoke probe (the pattern of
    skainet-backends/skainet-backend-jni-cpu/src/main/kotlin/sk/ainet/exec/kernel/jni/JniKernelProvider.kt:36-45)."""

    name = "cuda-sm100a"
    priority = 200   # scalar 0 / Panama 50 / native 100 (KernelProvider.kt:13-17)

    def __init__(self) -> None:
        self._available: Optional[bool] = None

    def isAvailable(self) -> bool:
        if self._available is None:
            try:
                probe = np.array([1.0, -2.5, 3.25], dtype=np.float32)
                out = np.zeros_like(probe)
                st = L.lib().skainet_cuda_smoke_double(_fp(probe), _fp(out), probe.size)
                self._available = st == L.OK and bool(np.array_equal(out, probe * 2))
            except (ImportError, OSError, AttributeError):
                self._available = False
        return self._available

    def matmulFp32(self):
        return None

    def matmulQ4K(self) -> Optional[CudaQ4KMatmulKernel]:
        return CudaQ4KMatmulKernel() if self.isAvailable() else None

    def matmulQ8_0(self) -> Optional[CudaQ8_0MatmulKernel]:
        return CudaQ8_0MatmulKernel() if self.isAvailable() else None

    def matmulQ6K(self) -> Optional[CudaQ6KMatmulKernel]:
        return CudaQ6KMatmulKernel() if self.isAvailable() else None

    def matmulQ5K(self) -> Optional[CudaQ5KMatmulKernel]:
        return CudaQ5KMatmulKernel() if self.isAvailable() else None

    def matmulQ6KRowMajor(self) -> Optional[CudaQ6KMatmulKernel]:
        return CudaQ6KMatmulKernel(row_major=True) if self.isAvailable() else None

    def matmulQ5KRowMajor(self) -> Optional[CudaQ5KMatmulKernel]:
        return CudaQ5KMatmulKernel(row_major=True) if self.isAvailable() else None

    def matmulQ4KRowMajor(self) -> Optional[CudaQ4KMatmulKernel]:
        return CudaQ4KMatmulKernel(row_major=True) if self.isAvailable() else None

    def matmulQ8_0RowMajor(self) -> Optional[CudaQ8_0MatmulKernel]:
        return CudaQ8_0MatmulKernel(row_major=True) if self.isAvailable() else None

    def normFp32(self) -> Optional[CudaFp32NormKernel]:
        return CudaFp32NormKernel() if self.isAvailable() else None

    def attentionFp32(self) -> Optional[CudaFp32AttentionKernel]:
        return CudaFp32AttentionKernel() if self.isAvailable() else None

    def softmaxFp32(self):
        return None

    def supports(self, opName: str, dtypeKeys: Sequence[str]) -> bool:
        """Same decision table as KernelProvider.supports (KernelProvider.kt:161-189)."""
        keys = list(dtypeKeys)
        if len(keys) == 1:
            if keys[0] != "Float32":
                return False
            if opName in ("layer_norm", "rms_norm"):
                return opName == "rms_norm" and self.normFp32() is not None
            if opName == "sdpa":
                return self.attentionFp32() is not None
            return False
        if len(keys) != 2 or keys[0] != "Float32" or opName != "matmul":
            return False
        return {"Q4_K": self.matmulQ4K, "Q8_0": self.matmulQ8_0, "Q6_K": self.matmulQ6K, "Q5_K": self.matmulQ5K}.get(keys[1], lambda: None)() is not None
