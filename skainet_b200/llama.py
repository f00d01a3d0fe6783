"""Host-side handle of the decoder runtime inside libskainet_cuda (include/skainet_cuda_llama.h)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import _lib as L
from .device import Weight

W_EMBED, W_HEAD, W_OUT_NORM, W_ATTN_NORM, W_Q, W_K, W_V, W_O, W_FFN_NORM, W_GATE, W_UP, W_DOWN, W_QKV, W_GATE_UP = range(14)


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn_dim", "vocab")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int32) for n in ("rope_mode", "max_seq", "max_batch", "linear_enc", "table_enc", "tp_rank", "tp_world")]


@dataclass
class LlamaConfig:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_dim: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 1e4
    rope_mode: int = 0
    max_seq: int = 1024
    max_batch: int = 1
    linear_enc: str = "Q4_K"
    table_enc: str = "Q8_0"
    tp_rank: int = 0
    tp_world: int = 1

    @classmethod
    def llama7b(cls, **kw) -> "LlamaConfig":
        """Llama-7B shape: 32 layers, d 4096, FFN 11008, 32 heads, vocab 32000; Q4_K linears, Q8_0 embed/output."""
        return cls(32, 4096, 32, 32, 128, 11008, 32000, **kw)

    @classmethod
    def llama70b(cls, **kw) -> "LlamaConfig":
        """Llama-70B-class shape: 80 layers, d 8192, FFN 28672, 64 q / 8 kv heads, vocab 128256, all Q4_K."""
        kw.setdefault("table_enc", "Q4_K")
        return cls(80, 8192, 64, 8, 128, 28672, 128256, **kw)

    def to_c(self) -> _Config:
        return _Config(self.n_layers, self.d_model, self.n_heads, self.n_kv_heads, self.head_dim, self.ffn_dim, self.vocab,
                       self.rms_eps, self.rope_theta, self.rope_mode, self.max_seq, self.max_batch, L.ENC[self.linear_enc],
                       L.ENC[self.table_enc], self.tp_rank, self.tp_world)


class Llama:
    def __init__(self, cfg: LlamaConfig):
        self.cfg = cfg
        h = C.c_int64()
        c = cfg.to_c()
        L.check(L.lib().skainet_cuda_llama_create(C.byref(c), C.byref(h)))
        self.handle = h.value

    # ---- weights --------------------------------------------------------------------------------
    def set_weight(self, layer: int, which: int, w: Weight) -> None:
        L.check(L.lib().skainet_cuda_llama_set_weight(self.handle, layer, which, w.handle))
        w.handle = 0      # the model owns it now

    def set_norm(self, layer: int, which: int, gamma: np.ndarray) -> None:
        g = np.ascontiguousarray(gamma, dtype=np.float32)
        assert g.size == self.cfg.d_model
        L.check(L.lib().skainet_cuda_llama_set_norm(self.handle, layer, which, g.ctypes.data_as(L.f32p)))

    def synth(self, seed: int = 100, std: float = 0.02) -> None:
        L.check(L.lib().skainet_cuda_llama_synth(self.handle, seed, std))

    def export_weight(self, layer: int, which: int) -> np.ndarray:
        """Canonical row-major packed bytes of this rank's shard of a tensor."""
        h = C.c_int64()
        L.check(L.lib().skainet_cuda_llama_get_weight(self.handle, layer, which, C.byref(h)))
        info = (C.c_int64 * 4)()
        L.check(L.lib().skainet_cuda_weight_info(h.value, info))
        out = np.empty(int(info[3]), dtype=np.uint8)
        L.check(L.lib().skainet_cuda_weight_export(h.value, out.ctypes.data_as(L.u8p), out.size))
        return out

    def weight(self, layer: int, which: int) -> Weight:
        """A borrowed view of a tensor the model owns (do not free)."""
        h = C.c_int64()
        L.check(L.lib().skainet_cuda_llama_get_weight(self.handle, layer, which, C.byref(h)))
        w = Weight(h.value)
        w.free = lambda: None      # borrowed
        return w

    def finalize(self) -> None:
        L.check(L.lib().skainet_cuda_llama_finalize(self.handle))

    @staticmethod
    def tp_unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        L.check(L.lib().skainet_cuda_llama_tp_unique_id(buf))
        return bytes(buf)

    def tp_init(self, unique_id: bytes) -> None:
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        L.check(L.lib().skainet_cuda_llama_tp_init(self.handle, buf))

    # ---- running ----------------------------------------------------------------------------------
    def reset(self) -> None:
        L.check(L.lib().skainet_cuda_llama_reset(self.handle))

    def prefill(self, tokens: Sequence[int], seq: int = 0, want_next: bool = True) -> Optional[int]:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        nxt = C.c_int32(-1)
        L.check(L.lib().skainet_cuda_llama_prefill(self.handle, seq, t.ctypes.data_as(L.i32p), t.size, C.byref(nxt) if want_next else None))
        return int(nxt.value) if want_next else None

    def fake_prefill(self, n: int, seq: int = 0, seed: int = 7) -> None:
        L.check(L.lib().skainet_cuda_llama_fake_prefill(self.handle, seq, n, seed))

    def decode(self, tokens_in: np.ndarray, tokens_out: np.ndarray) -> None:
        """One greedy step, host tokens in, host tokens out (int32 arrays of length batch; pinned for best latency)."""
        L.check(L.lib().skainet_cuda_llama_decode(self.handle, tokens_in.size, tokens_in.ctypes.data_as(L.i32p), tokens_out.ctypes.data_as(L.i32p)))

    def decode_ptr(self, batch: int, in_ptr: int, out_ptr: int) -> None:
        L.check(L.lib().skainet_cuda_llama_decode(self.handle, batch, C.cast(in_ptr, L.i32p), C.cast(out_ptr, L.i32p)))

    def generate(self, first_tokens: Sequence[int], n_steps: int) -> np.ndarray:
        """n_steps greedy steps on the device; returns [n_steps, batch] tokens."""
        first = np.ascontiguousarray(first_tokens, dtype=np.int32)
        out = np.empty((n_steps, first.size), dtype=np.int32)
        L.check(L.lib().skainet_cuda_llama_generate(self.handle, first.size, first.ctypes.data_as(L.i32p), n_steps, out.ctypes.data_as(L.i32p)))
        return out

    def logits(self, batch: int = 1) -> np.ndarray:
        out = np.empty((batch, self.cfg.vocab), dtype=np.float32)
        L.check(L.lib().skainet_cuda_llama_logits(self.handle, batch, out.ctypes.data_as(L.f32p)))
        return out

    def peek(self, which: int, n: int) -> np.ndarray:
        """Diagnostic read of an activation buffer (0 x, 1 q|k|v, 2 attention out, 3 gate|up, 4 q)."""
        out = np.empty(n, dtype=np.float32)
        L.check(L.lib().skainet_cuda_llama_peek(self.handle, which, out.ctypes.data_as(L.f32p), n))
        return out

    def tp_exchange_time(self, mode: int, rounds: int = 64, reps: int = 20) -> float:
        """Device microseconds of one group exchange of a [d_model] row, timed on its own (collective: all ranks call it).
        mode 0 peer-memory sum, 1 store + gather + sum + RMSNorm + quantize, 2 NCCL sum."""
        out = C.c_float()
        L.check(L.lib().skainet_cuda_llama_tp_exchange_time(self.handle, mode, rounds, reps, C.byref(out)))
        return float(out.value)

    def step_cost(self, batch: int = 1) -> tuple[int, int]:
        out = (C.c_int64 * 2)()
        L.check(L.lib().skainet_cuda_llama_step_cost(self.handle, batch, out))
        return int(out[0]), int(out[1])

    @property
    def stream(self) -> int:
        s = C.c_void_p()
        L.check(L.lib().skainet_cuda_llama_stream(self.handle, C.byref(s)))
        return s.value or 0

    def free(self) -> None:
        if self.handle:
            L.lib().skainet_cuda_llama_free(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
