"""CPU composer of a Llama-style decoder built only from the reference's operators — TEST
INFRASTRUCTURE ONLY (the oracle for greedy-token parity and the CPU baseline of the decode bench).

The reference repository has no transformer runtime (it lives in the sibling project
SKaiNET-transformers), so the model level is unpinned; what is pinned is every operator this file
calls: packed matvec, RMSNorm, SDPA and SiLU/mul/add go to the reference's own compiled C
(oracle/_ref) when it is present, else to the port; embedding rows use the bit-exact Q8_0/Q4_K
decoders; RoPE and arg max are the restatements in oracle/port.c. The KV cache holds binary16 values
(rounded to nearest even), converted back exactly for attention — what the CUDA backend stores.
"""
from __future__ import annotations

import numpy as np

from . import ref as R


class CpuLlama:
    def __init__(self, cfg, weights: dict, norms: dict | None = None, use_ref: bool | None = None, encs: dict | None = None):
        """cfg: an object with the fields of skainet_b200.llama.LlamaConfig. weights: {(layer, name): packed uint8}
        with names q,k,v,o,gate,up,down per layer and ('embed'), ('head') at layer -1. norms: {(layer, name): gamma}.
        encs: {(layer, name): encoding} for tensors whose encoding differs from the model's (a Q6_K tensor in a Q4_K model)."""
        self.cfg, self.w, self.norms, self.encs = cfg, weights, norms or {}, encs or {}
        self.use_ref = (R.ref() is not None) if use_ref is None else use_ref
        self.k = [[] for _ in range(cfg.n_layers)]
        self.v = [[] for _ in range(cfg.n_layers)]
        self.pos = 0
        self._embed = None

    def _gamma(self, layer, name):
        return self.norms.get((layer, name), np.ones(self.cfg.d_model, np.float32))

    def _mm(self, layer, name, x, rows, cols):
        enc = self.encs.get((layer, name), self.cfg.table_enc if name in ("embed", "head") else self.cfg.linear_enc)
        return R.matmul(enc, x, self.w[(layer, name)], cols, rows, "rm", use_ref=self.use_ref)

    def embed_row(self, token: int) -> np.ndarray:
        enc = self.encs.get((-1, "embed"), self.cfg.table_enc)
        bpr = self.cfg.d_model // R.BLOCK_ELEMS[enc]
        nb = R.BLOCK_BYTES[enc] * bpr
        return R.dequant(enc, self.w[(-1, "embed")][token * nb:(token + 1) * nb])

    def step(self, token: int) -> np.ndarray:
        """Feeds one token at the current position; returns the logits."""
        c = self.cfg
        D, H, HK = c.head_dim, c.n_heads, c.n_kv_heads
        x = self.embed_row(token)
        for l in range(c.n_layers):
            xn = R.rms_norm(x, self._gamma(l, "attn_norm"), c.rms_eps, use_ref=self.use_ref)
            q = self._mm(l, "q", xn, H * D, c.d_model)
            k = self._mm(l, "k", xn, HK * D, c.d_model)
            v = self._mm(l, "v", xn, HK * D, c.d_model)
            q = R.rope(q.reshape(H, D), H, D, self.pos, c.rope_theta, c.rope_mode)
            k = R.rope(k.reshape(HK, D), HK, D, self.pos, c.rope_theta, c.rope_mode)
            self.k[l].append(R.round_f16(k)); self.v[l].append(R.round_f16(v.reshape(HK, D)))
            K = np.stack(self.k[l], axis=1)[None]      # [1, HK, L, D]
            V = np.stack(self.v[l], axis=1)[None]
            a = R.sdpa(q.reshape(1, H, 1, D), K, V, 1.0 / np.sqrt(np.float32(D)), causal=True, use_ref=self.use_ref).reshape(-1)
            x = x + self._mm(l, "o", a, c.d_model, H * D)
            xn = R.rms_norm(x, self._gamma(l, "ffn_norm"), c.rms_eps, use_ref=self.use_ref)
            g = self._mm(l, "gate", xn, c.ffn_dim, c.d_model)
            u = self._mm(l, "up", xn, c.ffn_dim, c.d_model)
            x = x + self._mm(l, "down", R.swiglu(g, u), c.d_model, c.ffn_dim)
        self.pos += 1
        xn = R.rms_norm(x, self._gamma(-1, "out_norm"), c.rms_eps, use_ref=self.use_ref)
        return self._mm(-1, "head", xn, c.vocab, c.d_model)

    def greedy(self, prompt, n_new: int):
        """Runs the prompt token by token, then n_new greedy tokens. Returns (tokens, logits of every generated step)."""
        logits = None
        for t in prompt:
            logits = self.step(int(t))
        out, all_logits = [], []
        for _ in range(n_new):
            tok = R.argmax(logits)
            out.append(tok); all_logits.append(logits)
            logits = self.step(tok)
        return out, all_logits
