"""ctypes binding of libskainet_cuda.so — the same C ABI a JNI shim binds (include/skainet_cuda.h).

Loading fails loudly when the library is missing: there is no Python or CPU fallback for any kernel.
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libskainet_cuda.so")

OK = 0
ERR_INVALID, ERR_CUDA, ERR_NODEVICE, ERR_OOM, ERR_HANDLE, ERR_TIMEOUT, ERR_COMM = -1, -2, -3, -4, -5, -6, -7
ENC = {"Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}
ENC_NAME = {v: k for k, v in ENC.items()}
BLOCK_BYTES = {"Q8_0": 34, "Q4_K": 144, "Q5_K": 176, "Q6_K": 210}
BLOCK_ELEMS = {"Q8_0": 32, "Q4_K": 256, "Q5_K": 256, "Q6_K": 256}
ORDER_ROW_MAJOR, ORDER_INPUT_MAJOR = 0, 1
ACT_NATIVE, ACT_F32 = 0, 1

f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)
vp = C.c_void_p
i32, i64, f32 = C.c_int32, C.c_int64, C.c_float

_MATVEC = [f32p, i32, u8p, i32, i32, i32, f32p, i32]

# name -> argtypes; every entry returns int32 status unless listed in _RESTYPE.
SIGNATURES = {
    "skainet_cuda_last_error": [],
    "skainet_cuda_version": [],
    "skainet_cuda_device_count": [],
    "skainet_cuda_set_device": [i32],
    "skainet_cuda_device_info": [i64p],
    "skainet_cuda_device_status": [],
    "skainet_cuda_selftest_bounded_wait": [i32p],
    "skainet_cuda_smoke_double": [f32p, f32p, i32],
    "skainet_cuda_q4k_matmul": _MATVEC,
    "skainet_cuda_q4k_matmul_rm": _MATVEC,
    "skainet_cuda_q8_0_matmul": _MATVEC,
    "skainet_cuda_q8_0_matmul_rm": _MATVEC,
    "skainet_cuda_q6k_matmul": _MATVEC,
    "skainet_cuda_q6k_matmul_rm": _MATVEC,
    "skainet_cuda_q5k_matmul": _MATVEC,
    "skainet_cuda_q5k_matmul_rm": _MATVEC,
    "skainet_cuda_f32_rms_norm": [f32p, f32p, f32p, i32, i32, f32],
    "skainet_cuda_f32_sdpa": [f32p, f32p, f32p, f32p] + [i32] * 6 + [f32] + [i32] * 3 + [i32p, f32p] + [i32] * 4,
    "skainet_cuda_f32_unary": [i32, f32p, f32p, i32],
    "skainet_cuda_f32_binary": [i32, f32p, i32, f32p, i32, f32p, i32, i32],
    "skainet_cuda_dequant": [i32, u8p, i64, f32p],
    "skainet_cuda_malloc": [C.POINTER(vp), i64],
    "skainet_cuda_free": [vp],
    "skainet_cuda_memcpy_h2d": [vp, vp, i64, vp],
    "skainet_cuda_memcpy_d2h": [vp, vp, i64, vp],
    "skainet_cuda_stream_create": [C.POINTER(vp)],
    "skainet_cuda_stream_destroy": [vp],
    "skainet_cuda_stream_sync": [vp],
    "skainet_cuda_weight_upload": [u8p, i64, i32, i32, i32, i32, i64p],
    "skainet_cuda_weight_from_device": [vp, i64, i32, i32, i32, i32, i64p],
    "skainet_cuda_weight_synth": [i32, i32, i32, C.c_uint64, f32, i32, i64p],
    "skainet_cuda_weight_export": [i64, u8p, i64],
    "skainet_cuda_weight_info": [i64, i64p],
    "skainet_cuda_weight_free": [i64],
    "skainet_cuda_weight_dequant": [i64, vp, vp],
    "skainet_cuda_matmul_dev": [i64, vp, i32, vp, i32, vp],
    "skainet_cuda_probe_read_dev": [i64, vp],
    "skainet_cuda_matvec_fused_dev": [i64, vp, vp, f32, vp, vp, vp],
    "skainet_cuda_rms_norm_dev": [vp, vp, vp, i32, i32, f32, vp],
    "skainet_cuda_unary_dev": [i32, vp, vp, i64, vp],
    "skainet_cuda_binary_dev": [i32, vp, i32, vp, i32, vp, i64, i32, vp],
    "skainet_cuda_swiglu_dev": [vp, vp, vp, i64, vp],
    "skainet_cuda_rope_dev": [vp, vp, i32, i32, i32, f32, i32, vp],
    "skainet_cuda_argmax_dev": [vp, i32, i32, vp, vp],
    "skainet_cuda_embed_dev": [i64, vp, i32, vp, vp],
    "skainet_cuda_sdpa_dev": [vp, vp, vp, vp] + [i32] * 6 + [f32] + [i32] * 3 + [vp, vp] + [i32] * 4 + [vp],
    "skainet_cuda_attn_decode_dev": [vp, vp, vp, vp, i32, i32, i32, i32, i64, vp, i32, f32, i32, vp],
    "skainet_cuda_attn_decode_noalloc_dev": [vp, vp, vp, vp, i32, i32, i32, i32, i64, vp, i32, f32, i32, vp],
    "skainet_cuda_f32_to_f16_dev": [vp, vp, i64, vp],
    "skainet_cuda_weight_concat_rows": [i64, i64, i64, i64p],
    "skainet_cuda_fused_qkv_proj_dev": [i64, i32, i32, i32, vp, vp, f32, i32, vp, vp, vp, vp],
    "skainet_cuda_fused_swiglu_ffn_dev": [i64, i64, vp, vp, f32, i32, vp, vp, vp],
    "skainet_cuda_kv_create": [i32, i32, i32, i32, i32, i64p],
    "skainet_cuda_kv_create_turboquant": [i32, i32, i32, i32, i32, i32, i32, i32, i64p],
    "skainet_cuda_turboquant_encode": [f32p, i32, i32, i32, i32, u8p, f32p, u8p, f32p],
    "skainet_cuda_turboquant_decode": [u8p, f32p, u8p, C.c_float, i32, i32, i32, i32, f32p],
    "skainet_cuda_kv_free": [i64],
    "skainet_cuda_kv_append": [i64, i32, f32p, f32p],
    "skainet_cuda_kv_append_dev": [i64, i32, vp, vp, vp],
    "skainet_cuda_kv_read": [i64, i32, i32, i32, i32, f32p],
    "skainet_cuda_kv_evict": [i64, i32],
    "skainet_cuda_kv_clear": [i64],
    "skainet_cuda_kv_info": [i64, i64p],
    "skainet_cuda_kv_attn_decode_dev": [i64, i32, vp, vp, i32, i32, i32, f32, vp],
    # include/skainet_cuda_llama.h
    "skainet_cuda_llama_create": [vp, i64p],
    "skainet_cuda_llama_free": [i64],
    "skainet_cuda_llama_set_weight": [i64, i32, i32, i64],
    "skainet_cuda_llama_set_norm": [i64, i32, i32, f32p],
    "skainet_cuda_llama_synth": [i64, C.c_uint64, f32],
    "skainet_cuda_llama_get_weight": [i64, i32, i32, i64p],
    "skainet_cuda_llama_finalize": [i64],
    "skainet_cuda_llama_tp_unique_id": [C.POINTER(C.c_uint8)],
    "skainet_cuda_llama_tp_init": [i64, C.POINTER(C.c_uint8)],
    "skainet_cuda_llama_reset": [i64],
    "skainet_cuda_llama_prefill": [i64, i32, i32p, i32, i32p],
    "skainet_cuda_llama_fake_prefill": [i64, i32, i32, C.c_uint64],
    "skainet_cuda_llama_decode": [i64, i32, i32p, i32p],
    "skainet_cuda_llama_generate": [i64, i32, i32p, i32, i32p],
    "skainet_cuda_llama_logits": [i64, i32, f32p],
    "skainet_cuda_llama_step_cost": [i64, i32, i64p],
    "skainet_cuda_llama_peek": [i64, i32, f32p, i64],
    "skainet_cuda_llama_tp_exchange_time": [i64, i32, i32, i32, f32p],
    "skainet_cuda_llama_stream": [i64, C.POINTER(vp)],
}
_RESTYPE = {"skainet_cuda_last_error": C.c_char_p, "skainet_cuda_version": C.c_char_p}


class SkainetCudaError(RuntimeError):
    """A non-zero status from the library (status in ``.status``)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m skainet_b200.build` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    handle = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
        fn.argtypes = argtypes
        fn.restype = _RESTYPE.get(name, C.c_int32)
    return handle


def last_error() -> str:
    return lib().skainet_cuda_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise the Python counterpart of the Kotlin side's exceptions for a non-zero status."""
    if status == OK:
        return
    msg = last_error()
    if status == ERR_INVALID:
        raise ValueError(msg)          # IllegalArgumentException on the JVM
    if status == ERR_OOM:
        raise MemoryError(msg)
    raise SkainetCudaError(status, msg)
