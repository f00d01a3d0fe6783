"""Resident API over the C ABI: weights uploaded once, activations and KV cache in HBM.

Device pointers are plain integers (``DeviceBuffer.ptr``); a torch CUDA tensor's ``data_ptr()`` works
as well, which is how the bench harness shares buffers — the library itself never sees torch.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib as L


def set_device(device: int) -> None:
    L.check(L.lib().skainet_cuda_set_device(device))


def device_count() -> int:
    return int(L.lib().skainet_cuda_device_count())


def device_info() -> dict:
    out = (C.c_int64 * 4)()
    L.check(L.lib().skainet_cuda_device_info(out))
    return {"sm_count": out[0], "l2_bytes": out[1], "hbm_bytes": out[2], "cc": out[3]}


class DeviceBuffer:
    """A raw HBM allocation owned by the library."""

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        L.check(L.lib().skainet_cuda_malloc(C.byref(p), nbytes))
        self.ptr = p.value or 0
        self.nbytes = nbytes

    @classmethod
    def from_host(cls, a: np.ndarray, stream: int = 0) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes)
        buf.upload(a, stream)
        return buf

    def upload(self, a: np.ndarray, stream: int = 0) -> None:
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        L.check(L.lib().skainet_cuda_memcpy_h2d(self.ptr, a.ctypes.data, a.nbytes, stream))

    def download(self, dtype, count: int, stream: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        assert out.nbytes <= self.nbytes
        L.check(L.lib().skainet_cuda_memcpy_d2h(out.ctypes.data, self.ptr, out.nbytes, stream))
        return out

    def free(self) -> None:
        if self.ptr:
            L.lib().skainet_cuda_free(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Weight:
    """A packed [rows = out, cols = in] weight resident in HBM."""

    def __init__(self, handle: int):
        self.handle = handle
        info = (C.c_int64 * 4)()
        L.check(L.lib().skainet_cuda_weight_info(handle, info))
        self.encoding = L.ENC_NAME[info[0]]
        self.rows, self.cols, self.packed_bytes = int(info[1]), int(info[2]), int(info[3])

    @classmethod
    def upload(cls, packed: np.ndarray, encoding: str, rows: int, cols: int, order: int = L.ORDER_ROW_MAJOR) -> "Weight":
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        h = C.c_int64()
        L.check(L.lib().skainet_cuda_weight_upload(packed.ctypes.data_as(L.u8p), packed.size, L.ENC[encoding], rows, cols,
                                                   order, C.byref(h)))
        return cls(h.value)

    @classmethod
    def from_device(cls, dev_ptr: int, nbytes: int, encoding: str, rows: int, cols: int,
                    order: int = L.ORDER_ROW_MAJOR) -> "Weight":
        h = C.c_int64()
        L.check(L.lib().skainet_cuda_weight_from_device(dev_ptr, nbytes, L.ENC[encoding], rows, cols, order, C.byref(h)))
        return cls(h.value)

    @classmethod
    def synth(cls, encoding: str, rows: int, cols: int, seed: int, std: float = 0.02, mode: int = 0) -> "Weight":
        h = C.c_int64()
        L.check(L.lib().skainet_cuda_weight_synth(L.ENC[encoding], rows, cols, seed, std, mode, C.byref(h)))
        return cls(h.value)

    def export(self) -> np.ndarray:
        out = np.empty(self.packed_bytes, dtype=np.uint8)
        L.check(L.lib().skainet_cuda_weight_export(self.handle, out.ctypes.data_as(L.u8p), out.size))
        return out

    def dequant(self) -> np.ndarray:
        buf = DeviceBuffer(self.rows * self.cols * 4)
        L.check(L.lib().skainet_cuda_weight_dequant(self.handle, buf.ptr, 0))
        out = buf.download(np.float32, self.rows * self.cols).reshape(self.rows, self.cols)
        buf.free()
        return out

    def free(self) -> None:
        if self.handle:
            L.lib().skainet_cuda_weight_free(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def matmul(w: Weight, x_ptr: int, m: int, y_ptr: int, act_mode: int = L.ACT_NATIVE, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_matmul_dev(w.handle, x_ptr, m, y_ptr, act_mode, stream))


def matvec_fused(w: Weight, x_ptr: int, gamma_ptr: int, eps: float, resid_ptr: int, y_ptr: int, stream: int = 0) -> None:
    """y = (resid +) W . quantize(rmsnorm(x) if gamma else x), one launch."""
    L.check(L.lib().skainet_cuda_matvec_fused_dev(w.handle, x_ptr, gamma_ptr or None, eps, resid_ptr or None, y_ptr, stream))


def matmul_host(w: Weight, x: np.ndarray, act_mode: int = L.ACT_NATIVE) -> np.ndarray:
    """Convenience: x [m, cols] (host) -> y [m, rows] (host) through device buffers."""
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, w.cols)
    m = x2.shape[0]
    dx = DeviceBuffer.from_host(x2)
    dy = DeviceBuffer(max(4, m * w.rows * 4))
    matmul(w, dx.ptr, m, dy.ptr, act_mode)
    y = dy.download(np.float32, m * w.rows).reshape(m, w.rows)
    dx.free(); dy.free()
    return y if x.ndim > 1 else y[0]


def rms_norm(in_ptr: int, gamma_ptr: int, out_ptr: int, rows: int, cols: int, eps: float, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_rms_norm_dev(in_ptr, gamma_ptr, out_ptr, rows, cols, eps, stream))


def swiglu(gate_ptr: int, up_ptr: int, out_ptr: int, n: int, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_swiglu_dev(gate_ptr, up_ptr, out_ptr, n, stream))


def rope(x_ptr: int, pos_ptr: int, rows: int, heads: int, head_dim: int, theta: float = 1e4, mode: int = 0,
         stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_rope_dev(x_ptr, pos_ptr, rows, heads, head_dim, theta, mode, stream))


def argmax(x_ptr: int, rows: int, cols: int, out_ptr: int, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_argmax_dev(x_ptr, rows, cols, out_ptr, stream))


def embed(table: Weight, ids_ptr: int, n: int, out_ptr: int, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_embed_dev(table.handle, ids_ptr, n, out_ptr, stream))


def f32_to_f16(in_ptr: int, out_ptr: int, n: int, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_f32_to_f16_dev(in_ptr, out_ptr, n, stream))


def attn_decode(q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int, batch: int, heads: int, kv_heads: int, head_dim: int,
                cache_stride: int, kv_len_ptr: int, max_kv_len: int, scale: float, window: int = 0, stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_attn_decode_dev(q_ptr, k_ptr, v_ptr, out_ptr, batch, heads, kv_heads, head_dim,
                                                 cache_stride, kv_len_ptr, max_kv_len, scale, window, stream))


def sync(stream: int = 0) -> None:
    L.check(L.lib().skainet_cuda_stream_sync(stream))


def attn_decode_noalloc(q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int, batch: int, heads: int, kv_heads: int, head_dim: int,
                        cache_stride: int, kv_len_ptr: int, max_kv_len: int, scale: float, window: int = 0, stream: int = 0) -> None:
    """attn_decode for hosts that must not allocate: split-K partials in the library's built-in 4 MiB area.
    Raises ValueError when the problem does not fit it. Calls that overlap on the GPU race on that area."""
    L.check(L.lib().skainet_cuda_attn_decode_noalloc_dev(q_ptr, k_ptr, v_ptr, out_ptr, batch, heads, kv_heads, head_dim,
                                                         cache_stride, kv_len_ptr, max_kv_len, scale, window, stream))


def concat_rows(a: Weight, b: Weight, c: Optional[Weight] = None) -> Weight:
    """Rows of a, b (and c) as one new resident weight (merged q|k|v or gate|up); the parts stay valid."""
    h = C.c_int64()
    L.check(L.lib().skainet_cuda_weight_concat_rows(a.handle, b.handle, c.handle if c is not None else 0, C.byref(h)))
    return Weight(h.value)


def fused_qkv_proj(w_qkv: Weight, q_rows: int, k_rows: int, v_rows: int, x_ptr: int, m: int, q_ptr: int, k_ptr: int, v_ptr: int,
                   gamma_ptr: int = 0, eps: float = 0.0, stream: int = 0) -> None:
    """The graph-level fused op `fused_qkv_proj` (optionally with the RMSNorm that feeds it)."""
    L.check(L.lib().skainet_cuda_fused_qkv_proj_dev(w_qkv.handle, q_rows, k_rows, v_rows, x_ptr, gamma_ptr or None, eps, m, q_ptr, k_ptr,
                                                    v_ptr, stream))


def fused_swiglu_ffn(w_gate_up: Weight, w_down: Weight, x_ptr: int, m: int, out_ptr: int, resid_ptr: int = 0, gamma_ptr: int = 0,
                     eps: float = 0.0, stream: int = 0) -> None:
    """The graph-level fused op `fused_swiglu_ffn`: out = (resid +) down(silu(gate(x)) * up(x)), optionally normalised first."""
    L.check(L.lib().skainet_cuda_fused_swiglu_ffn_dev(w_gate_up.handle, w_down.handle, x_ptr, gamma_ptr or None, eps, m, resid_ptr or None,
                                                      out_ptr, stream))
