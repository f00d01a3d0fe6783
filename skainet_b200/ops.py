"""Resident-activation ops over the C ABI: the host-side mirror of the ops class a CUDA backend registers in front of
the CPU ops (the pattern of the browser tier's ops class,
skainet-backends/skainet-backend-wasm-simd/src/wasmJsMain/kotlin/sk/ainet/exec/wasm/WasmCpuOps.kt:18-50,92-117):
the outputs of matmul / norm / attention / elementwise ops stay in HBM as `DeviceTensor`s (the counterpart of
`Storage.Device`, skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/memory/Storage.kt:129-136,230), and
`copyFrom` / `copyInto` are the only host crossings. `CudaOps.host_crossings` counts them, so a test (or a caller) can
check that a chain of ops made none. Method names follow TensorOps / FusedNormOps of the reference."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib as L
from .device import DeviceBuffer, Weight

UNARY = {"relu": 0, "sigmoid": 1, "silu": 2, "gelu": 3, "geluErf": 4, "erf": 5, "tanh": 6}
BINARY = {"add": 0, "subtract": 1, "multiply": 2, "divide": 3}


class DeviceTensor:
    """A dense fp32 tensor resident in HBM (row-major)."""

    def __init__(self, ops: "CudaOps", shape: Sequence[int], buf: Optional[DeviceBuffer] = None):
        self.ops, self.shape = ops, tuple(int(d) for d in shape)
        self.volume = int(np.prod(self.shape)) if self.shape else 1
        self.buf = buf if buf is not None else DeviceBuffer(max(4, self.volume * 4))

    @property
    def ptr(self) -> int:
        return self.buf.ptr

    def copyFrom(self, host: np.ndarray) -> "DeviceTensor":
        a = np.ascontiguousarray(host, dtype=np.float32)
        assert a.size == self.volume
        self.buf.upload(a, self.ops.stream)
        self.ops.host_crossings += 1
        return self

    def copyInto(self, host: Optional[np.ndarray] = None) -> np.ndarray:
        out = self.buf.download(np.float32, self.volume, self.ops.stream).reshape(self.shape)
        self.ops.host_crossings += 1
        if host is not None:
            host[...] = out
            return host
        return out


class CudaOps:
    """matmul over packed weights, RMSNorm, attention and elementwise ops on resident tensors."""

    def __init__(self, stream: int = 0):
        self.stream = stream
        self.host_crossings = 0

    # ---- tensors ------------------------------------------------------------------------------------------
    def tensor(self, host: np.ndarray) -> DeviceTensor:
        return DeviceTensor(self, np.shape(host)).copyFrom(host)

    def empty(self, *shape: int) -> DeviceTensor:
        return DeviceTensor(self, shape)

    # ---- matmul over a packed [out, in] weight: y = x . W^T ---------------------------------------------------
    def matmul(self, x: DeviceTensor, w: Weight, act_mode: int = L.ACT_NATIVE) -> DeviceTensor:
        if x.shape[-1] != w.cols:
            raise ValueError(f"matmul: activation inner dimension {x.shape[-1]} != weight inputDim {w.cols}")
        m = x.volume // w.cols
        out = DeviceTensor(self, x.shape[:-1] + (w.rows,))
        L.check(L.lib().skainet_cuda_matmul_dev(w.handle, x.ptr, m, out.ptr, act_mode, self.stream))
        return out

    matmulWeightTransposed = matmul

    # ---- FusedNormOps.rmsNorm ----------------------------------------------------------------------------------------
    def rmsNorm(self, x: DeviceTensor, gamma: Optional[DeviceTensor], eps: float = 1e-5) -> DeviceTensor:
        cols = x.shape[-1]
        out = DeviceTensor(self, x.shape)
        L.check(L.lib().skainet_cuda_rms_norm_dev(x.ptr, gamma.ptr if gamma is not None else None, out.ptr, x.volume // cols, cols, eps, self.stream))
        return out

    # ---- elementwise -----------------------------------------------------------------------------------------------------
    def _unary(self, name: str, x: DeviceTensor) -> DeviceTensor:
        out = DeviceTensor(self, x.shape)
        L.check(L.lib().skainet_cuda_unary_dev(UNARY[name], x.ptr, out.ptr, x.volume, self.stream))
        return out

    def _binary(self, name: str, a: DeviceTensor, b: DeviceTensor) -> DeviceTensor:
        # operand modes of the reference kernel: 0 full, 1 scalar, 2 bias over the innermost dimension
        if b.volume == a.volume:
            mode, inner = 0, 1
        elif b.volume == 1:
            mode, inner = 1, 1
        elif b.volume == a.shape[-1]:
            mode, inner = 2, a.shape[-1]
        else:
            raise ValueError(f"{name}: shapes {a.shape} and {b.shape} do not broadcast (full, scalar or innermost bias)")
        out = DeviceTensor(self, a.shape)
        L.check(L.lib().skainet_cuda_binary_dev(BINARY[name], a.ptr, 0, b.ptr, mode, out.ptr, a.volume, inner, self.stream))
        return out

    def add(self, a, b): return self._binary("add", a, b)
    def subtract(self, a, b): return self._binary("subtract", a, b)
    def multiply(self, a, b): return self._binary("multiply", a, b)
    def divide(self, a, b): return self._binary("divide", a, b)
    def relu(self, x): return self._unary("relu", x)
    def sigmoid(self, x): return self._unary("sigmoid", x)
    def silu(self, x): return self._unary("silu", x)
    def gelu(self, x): return self._unary("gelu", x)
    def tanh(self, x): return self._unary("tanh", x)

    # ---- ops.scaledDotProductAttention (TensorOps.kt:410-458) -------------------------------------------------------------
    def scaledDotProductAttention(self, q: DeviceTensor, k: DeviceTensor, v: DeviceTensor, scale: float = 0.0, causal: bool = False,
                                  window: int = 0, rightContext: int = 0) -> DeviceTensor:
        B, H, Sq, D = q.shape
        Bk, Hkv, Skv, Dk = k.shape
        if (Bk, Dk) != (B, D) or v.shape != k.shape or H % Hkv:
            raise ValueError(f"scaledDotProductAttention: q {q.shape}, k {k.shape}, v {v.shape}")
        out = DeviceTensor(self, q.shape)
        sc = scale if scale != 0.0 else float(1.0 / np.sqrt(D))
        L.check(L.lib().skainet_cuda_sdpa_dev(q.ptr, k.ptr, v.ptr, out.ptr, B, H, Hkv, Sq, Skv, D, sc, 1 if causal else 0, window, rightContext,
                                              None, None, 0, 0, 0, 0, self.stream))
        return out

    # ---- gather over a packed table, arg max ----------------------------------------------------------------------------
    def gather(self, table: Weight, ids: np.ndarray) -> DeviceTensor:
        idx = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        d_ids = DeviceBuffer.from_host(idx, self.stream)       # indices are inputs of the op, like a token id: not an activation crossing
        out = DeviceTensor(self, (idx.size, table.cols))
        L.check(L.lib().skainet_cuda_embed_dev(table.handle, d_ids.ptr, idx.size, out.ptr, self.stream))
        L.check(L.lib().skainet_cuda_stream_sync(self.stream))
        d_ids.free()
        return out

    def argMax(self, x: DeviceTensor) -> np.ndarray:
        cols = x.shape[-1]
        rows = x.volume // cols
        d_out = DeviceBuffer(4 * rows)
        L.check(L.lib().skainet_cuda_argmax_dev(x.ptr, rows, cols, d_out.ptr, self.stream))
        self.host_crossings += 1
        return d_out.download(np.int32, rows, self.stream)
