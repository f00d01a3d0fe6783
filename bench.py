#!/usr/bin/env python
"""Benchmark of the packed-quantized decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0). Workloads (all inputs synthetic and seeded):

  decode_70b (default) — benchmark config 5: Llama-style 80 layers, d 8192, FFN 28672, 64 q / 8 kv
      heads, vocab 128256, all Q4_K, random-init N(0,0.02) packed on the device; greedy decode at
      batch 1 behind a 4096-token context, tensor-parallel over the N GPUs (strong scaling: the same
      model and batch at every N). metric = decode tokens/s. A step is one decode step (one token per
      sequence). The context's K/V are seeded noise, not a real prefill (the reference has no batched
      GEMM, so a 4096-row prompt is out of reach for its side). --batch B decodes B sequences.
  decode_7b — benchmark config 4: 32 layers, d 4096, FFN 11008, 32 heads, vocab 32000; Q4_K linears,
      Q8_0 embedding/output; batch 1 behind a 512-token context.
  decode_7b_mixed — decode_7b with attn_v and ffn_down of every second layer as Q6_K (the mix K-quant files carry);
      one GPU.
  q4k_matvec — benchmark config 2 at M=1: W[11008,4096] and W[4096,11008]; metric = algorithmic HBM
      GB/s over a sweep of distinct weights larger than 2x L2.
  q8_0_matvec — benchmark config 1: Q8_0 W[4096,4096], same protocol.
  q6k_matvec, q5k_matvec — config 2's two shapes in the encodings Q4_K_M / Q5_K_M files mix in, same protocol.
  q6k_gemm, q5k_gemm — the q4k_gemm protocol (--batch activation rows, default 512) on the same shapes as Q6_K / Q5_K.
  attn_decode — benchmark config 3: GQA decode attention, 32 query / 8 KV heads, head_dim 128, f16 cache of
      --context keys (default 4096) for --batch sequences; metric = K/V bytes read per second.
  generate_7b — benchmark config 4 as one request: 512 random prompt tokens through the real prefill, then 128 greedy
      tokens; metric = generated tokens per second of request time, with the two phases reported apart.
  q4k_gemm — benchmark config 2 at M = --batch rows (default 512) through the tensor-core tile kernels (tcgen05 from 288 rows);
      metric = 2*M*rows*cols operations per second, roofline against the measured cuBLAS bf16 burst.
  tp_collective — N >= 2 ranks: nothing but the group exchanges of a decode step (one [8192] fp32 row), timed on their own
      in a CUDA graph: the peer-memory sum, the store + gather + sum + RMSNorm + quantize kernel, and ncclAllReduce of the
      same row; metric = microseconds per exchange (lower is better). The N > 1 decode lines carry the same three numbers
      under `tp_exchange`.
  kv_turboquant — the TurboQuant KV store (4-bit keys and values, 8 heads x 128, 32 layers): one decode step of attention over
      --context positions per layer (blocks decoded to fp32, then fp32 attention); metric = microseconds per call (lower is better).

`value` is timed on the device with everything resident in HBM (decode: one CUDA-graph replay per
step, tokens fed back on the device). `e2e` is the same metric through the C ABI with HOST buffers
(decode: one `skainet_cuda_llama_decode` call per step, token ids host -> device and back, host
synchronisation every step; matvec: activation in, output out per call, weights resident).
`roofline.frac` is the whole step (bytes a step must read / step time); `roofline.kernel_*` is the dequant-fused matvec
path measured live over the workload's own weights.
`--impl reference` times the reference's own C kernels (oracle/_ref; the port if absent) on the host:
for decode a CPU composer built from those kernels, measured on a bounded number of layers and scaled.
PyTorch is used here for events, pinned memory and the process group only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MATVEC_WORKLOADS = {
    # name: (encoding, [(rows=out, cols=in), ...], block bytes, block elems)
    "q4k_matvec": ("Q4_K", [(11008, 4096), (4096, 11008)], 144, 256),
    "q8_0_matvec": ("Q8_0", [(4096, 4096)], 34, 32),
    # the formats Q4_K_M / Q5_K_M files mix in (ffn_down, attn_v, output head): config 2's shapes in those encodings
    "q6k_matvec": ("Q6_K", [(11008, 4096), (4096, 11008)], 210, 256),
    "q5k_matvec": ("Q5_K", [(11008, 4096), (4096, 11008)], 176, 256),
}
DECODE_WORKLOADS = {"decode_70b": ("70b", 4096), "decode_7b": ("7b", 512), "decode_7b_mixed": ("7b", 512)}
# a K-quant file's usual mix: attn_v and ffn_down of every second layer carried as Q6_K beside the Q4_K tensors
MIXED_WORKLOADS = {"decode_7b_mixed"}
# decode attention alone: (query heads, kv heads, head_dim); context from --context
ATTN_WORKLOADS = {"attn_decode": (32, 8, 128)}
# batched rows through the tensor-core tile kernel: the Q4_K sweep shapes with --batch activation rows (default 512)
GEMM_WORKLOADS = {"q4k_gemm": [(11008, 4096), (4096, 11008)], "q6k_gemm": [(11008, 4096), (4096, 11008)], "q5k_gemm": [(11008, 4096), (4096, 11008)]}
GEMM_ENC = {"q4k_gemm": "Q4_K", "q6k_gemm": "Q6_K", "q5k_gemm": "Q5_K"}
# whole requests: (model, prompt tokens, generated tokens)
REQUEST_WORKLOADS = {"generate_7b": ("7b", 512, 128)}
BLOCK = {"Q4_K": (144, 256), "Q8_0": (34, 32), "Q5_K": (176, 256), "Q6_K": (210, 256)}


def algorithmic_bytes(enc_bytes: int, enc_elems: int, rows: int, cols: int, m: int = 1) -> int:
    """Bytes one matvec must move: packed weight once, activation in, output out (fp32)."""
    return rows * (cols // enc_elems) * enc_bytes + 4 * m * (rows + cols)


# DRAM bytes (read + write) per algorithmic byte of the weight-streaming matvec kernels, from ncu captures of
# q4k_matvec_ring_kernel: 25.387 MB per 11008x4096 launch against 25.362 MB algorithmic, 264.27 MB per
# 57344x8192 launch against 264.24 MB.  Traffic grows in proportion to the weight bytes (each byte is read once).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.001


def load_tensor_peak() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["bf16_tflops"]), "measured (cuBLAS bf16 burst)"
    return 1590.0, "fallback"


def load_peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        ok = [r for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        sm = [float(r[0]) for r in ok]
        mx = [float(r[1]) for r in ok if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in ok for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def model_config(name: str, **kw):
    from skainet_b200.llama import LlamaConfig
    return LlamaConfig.llama70b(**kw) if name == "70b" else LlamaConfig.llama7b(**kw)


# ---------------------------------------------------------------------------------------------------
# CPU side: the reference's own C kernels on the host cores
# ---------------------------------------------------------------------------------------------------
def random_blocks(rng, enc: str, rows: int, cols: int) -> np.ndarray:
    """Random valid packed blocks (random codes/scales, sane f16 fields), the reference's microbench fixture style."""
    bb, be = BLOCK[enc]
    packed = rng.integers(0, 256, size=rows * (cols // be) * bb, dtype=np.uint8)
    blk = packed.reshape(-1, bb)
    if enc == "Q6_K":                       # ql[128] | qh[64] | scales[16] | d
        blk[:, 208:210] = np.array([0.0002], np.float16).view(np.uint8)
        return packed
    blk[:, 0:2] = np.array([0.002], np.float16).view(np.uint8)
    if enc in ("Q4_K", "Q5_K"):
        blk[:, 2:4] = np.array([0.002], np.float16).view(np.uint8)
    return packed


def cpu_matvec_rate(workload: str, seconds: float) -> dict:
    from oracle import ref as R
    enc, shapes, bb, be = MATVEC_WORKLOADS[workload]
    use_ref = R.ref() is not None
    rng = np.random.default_rng(5)
    items = [(r, c, random_blocks(rng, enc, r, c), rng.standard_normal(c).astype(np.float32)) for r, c in shapes]
    for r, c, packed, x in items:
        R.matmul(enc, x, packed, c, r, "rm", use_ref=use_ref)
    t0 = time.perf_counter(); done = 0; calls = 0
    while time.perf_counter() - t0 < seconds:
        for r, c, packed, x in items:
            R.matmul(enc, x, packed, c, r, "rm", use_ref=use_ref)
            done += algorithmic_bytes(bb, be, r, c); calls += 1
    dt = time.perf_counter() - t0
    fn = "skainet_%s_matmul_rm" % {"Q4_K": "q4k", "Q8_0": "q8_0", "Q6_K": "q6k", "Q5_K": "q5k"}[enc]
    return {"value": done / dt / 1e9, "unit": "GB/s", "cores": 4 if use_ref else 1, "kind": "reference" if use_ref else "port",
            "sample": f"{calls} calls of {fn if use_ref else 'the oracle port'} over the workload's {len(items)} shapes in {dt:.1f} s "
                      f"({'its 4-thread row pool' if use_ref else 'scalar'}; host has {os.cpu_count()} cores)", "seconds": dt}


def cpu_decode_rate(model: str, ctx: int, budget_s: float, mixed: bool = False) -> dict:
    """tokens/s of a decoder composed from the reference's C kernels: one layer (random valid packed
    weights of the model's shapes, context of `ctx` cached keys) and the output head are timed, the layer
    time is multiplied by the layer count. Activation quantization, RMSNorm, SDPA, SiLU, mul, add as the
    reference computes them; 4 threads (the library's own cap)."""
    from oracle import ref as R
    cfg = model_config(model)
    use_ref = R.ref() is not None
    rng = np.random.default_rng(7)
    D, H, HK, d, F = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_model, cfg.ffn_dim
    le, te = cfg.linear_enc, cfg.table_enc
    W = {"q": (H * D, d), "k": (HK * D, d), "v": (HK * D, d), "o": (d, H * D), "gate": (F, d), "up": (F, d), "down": (d, F)}
    packed = {k: random_blocks(rng, le, r, c) for k, (r, c) in W.items()}
    packed6 = {k: random_blocks(rng, "Q6_K", *W[k]) for k in ("v", "down")} if mixed else {}
    vocab_sample = min(cfg.vocab, 16000)          # the head is timed on a slice of its rows and scaled
    head = random_blocks(rng, te, vocab_sample, d)
    K = rng.standard_normal((1, HK, ctx + 1, D)).astype(np.float16).astype(np.float32)
    V = rng.standard_normal((1, HK, ctx + 1, D)).astype(np.float16).astype(np.float32)
    x = rng.standard_normal(d).astype(np.float32)
    ones = np.ones(d, np.float32)

    def mm(name, v, q6=False):
        r, c = W[name]
        if q6 and name in packed6:
            return R.matmul("Q6_K", v, packed6[name], c, r, "rm", use_ref=use_ref)
        return R.matmul(le, v, packed[name], c, r, "rm", use_ref=use_ref)

    def layer(x, q6=False):
        xn = R.rms_norm(x, ones, cfg.rms_eps, use_ref=use_ref)
        q = R.rope(mm("q", xn).reshape(H, D), H, D, ctx); k = R.rope(mm("k", xn).reshape(HK, D), HK, D, ctx); v = mm("v", xn, q6)
        K[0, :, ctx] = R.round_f16(k); V[0, :, ctx] = R.round_f16(v.reshape(HK, D))
        a = R.sdpa(q.reshape(1, H, 1, D), K, V, 1.0 / np.sqrt(D), causal=True, use_ref=use_ref).reshape(-1)
        x = x + mm("o", a)
        xn = R.rms_norm(x, ones, cfg.rms_eps, use_ref=use_ref)
        return x + mm("down", R.swiglu(mm("gate", xn), mm("up", xn)), q6)

    layer(x)                                        # warm-up
    t0 = time.perf_counter(); n_layer = 0
    # mixed: layers with Q6_K attn_v / ffn_down and plain ones alternate, an even number of them is timed
    while n_layer < 1 or (mixed and n_layer % 2 == 1) or time.perf_counter() - t0 < budget_s * 0.8:
        x = layer(x, mixed and n_layer % 2 == 0); x /= max(1.0, float(np.abs(x).max())); n_layer += 1
    t_layer = (time.perf_counter() - t0) / n_layer
    t0 = time.perf_counter(); n_head = 0
    while n_head < 1 or time.perf_counter() - t0 < budget_s * 0.2:
        R.matmul(te, R.rms_norm(x, ones, cfg.rms_eps, use_ref=use_ref), head, d, vocab_sample, "rm", use_ref=use_ref); n_head += 1
    t_head = (time.perf_counter() - t0) / n_head * (cfg.vocab / vocab_sample)
    t_tok = t_layer * cfg.n_layers + t_head
    return {"value": 1.0 / t_tok, "unit": "tokens/s", "cores": 4 if use_ref else 1, "kind": "reference" if use_ref else "port",
            "sample": f"{n_layer} decoder layer(s) and {n_head} output-head pass(es) on {vocab_sample} of {cfg.vocab} rows, composed from "
                      f"{'the reference C kernels (4-thread row pool)' if use_ref else 'the oracle port (scalar)'}; per-layer {t_layer * 1e3:.1f} ms x "
                      f"{cfg.n_layers} layers + head {t_head * 1e3:.1f} ms, extrapolated; host has {os.cpu_count()} cores",
            "seconds": t_tok}


def cpu_attn_rate(workload: str, ctx: int, batch: int) -> dict:
    """The reference's fused fp32 SDPA (skainet_f32_sdpa, one query row per head) on the same shape; the
    rate is quoted on the f16 cache bytes the GPU path reads, so the two are comparable."""
    from oracle import ref as R
    h, hkv, d = ATTN_WORKLOADS[workload]
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, h, 1, d), dtype=np.float32)
    k = rng.standard_normal((1, hkv, ctx, d), dtype=np.float32)
    v = rng.standard_normal((1, hkv, ctx, d), dtype=np.float32)
    use_ref = R.ref() is not None
    R.sdpa(q, k, v, d ** -0.5, causal=False, use_ref=use_ref)
    t0 = time.perf_counter(); n = 0
    while time.perf_counter() - t0 < 3.0:
        R.sdpa(q, k, v, d ** -0.5, causal=False, use_ref=use_ref); n += 1
    dt = (time.perf_counter() - t0) / n
    return {"value": 2 * hkv * ctx * d * 2 / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "reference" if use_ref else "port",
            "sample": f"one sequence of the batch, fp32 K/V on the host, {n} calls", "seconds": dt * n}


def run_reference(args) -> None:
    rank, _, _ = dist_env()
    if rank != 0:
        return
    budget = max(2.0, min(20.0, 90.0 / max(1, args.steps + args.warmup)))
    vals, times = [], []
    for i in range(args.warmup + args.steps):
        if args.workload in MATVEC_WORKLOADS:
            r = cpu_matvec_rate(args.workload, budget); unit = "GB/s"; metric = f"{args.workload}_hbm_gbs"
        elif args.workload in ATTN_WORKLOADS:
            r = cpu_attn_rate(args.workload, args.context, max(1, args.batch)); unit = "GB/s"; metric = "attn_decode_hbm_gbs"
        elif args.workload in GEMM_WORKLOADS:
            r = cpu_gemm_rate(args.workload, args.batch if args.batch > 1 else 512, budget); unit = "TFLOP/s"; metric = f"{args.workload}_tflops"
        elif args.workload in REQUEST_WORKLOADS:
            r = cpu_request_rate(args.workload, budget); unit = "tokens/s"; metric = "request_generated_tokens_per_s"
        else:
            model, ctx = DECODE_WORKLOADS[args.workload]
            r = cpu_decode_rate(model, ctx, budget, mixed=args.workload in MIXED_WORKLOADS); unit = "tokens/s"; metric = "decode_tokens_per_s"
        if i >= args.warmup:
            vals.append(r["value"]); times.append(r["seconds"] * 1e3)
    v = float(np.mean(vals))
    line = {"impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": float(np.mean(times)), "higher_is_better": True,
            "scaling": "weak" if args.workload in MATVEC_WORKLOADS else "strong", "vs_baseline": None, "dtype": dtype_of(args.workload),
            "data": "synthetic", "config": workload_config(args, 1, {"weights": "random valid packed blocks on the host (the integer kernels' time does not depend on the values)",
                                                                     "context_fill": "random f16-rounded K/V on the host" }),
            "cpu_baseline": {"value": v, "unit": unit, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def dtype_of(workload: str) -> str:
    if workload == "q6k_gemm":
        return "s8 (6-bit code - 32) x s8 -> s32 on mma.sync per 16-element scale group, int8 group scales, f32 block terms"
    if workload == "q5k_gemm":
        return "f16 (5-bit code x 6-bit scale, exact) x f32 activation as two f16 terms -> f32 on mma.sync"
    if workload in GEMM_WORKLOADS:
        return "f16 (4-bit code x 6-bit scale, exact) x f16 (int8 code) -> f32 on tcgen05 for m >= 288; u8 x s8 -> s32 on mma.sync below"
    if workload in ATTN_WORKLOADS:
        return "f16 K/V, f32 q split in two f16 terms, f32 accumulate"
    if workload == "q8_0_matvec":
        return "int8 x int8 (two-term activation) -> int32, f32 accumulate"
    if workload in MIXED_WORKLOADS:
        return "int8 x int4 / int6 -> int32, f32 accumulate (attention and norms f32, KV f16)"
    if workload == "q6k_matvec":
        return "int8 x int6 -> int32, f32 accumulate"
    if workload == "q5k_matvec":
        return "f32 x 5-bit code, f32 accumulate"
    return "int8 x int4 -> int32, f32 accumulate (attention and norms f32, KV f16)" if workload in DECODE_WORKLOADS \
        else "int8 x int4 -> int32, f32 accumulate"


def workload_config(args, world: int, extra: dict | None = None) -> dict:
    if args.workload in REQUEST_WORKLOADS:
        model, n_prompt, n_gen = REQUEST_WORKLOADS[args.workload]
        cfg = model_config(model)
        c = {"workload": args.workload, "layers": cfg.n_layers, "d_model": cfg.d_model, "ffn": cfg.ffn_dim, "heads": cfg.n_heads,
             "kv_heads": cfg.n_kv_heads, "vocab": cfg.vocab, "linear": "Q4_K", "tables": "Q8_0", "batch": 1, "prompt_tokens": n_prompt,
             "generated_tokens": n_gen, "prompt": "uniform random token ids, seeded", "weights": "N(0,0.02) packed on device, seeded",
             "l2": "weights per pass far larger than L2"}
    elif args.workload in GEMM_WORKLOADS:
        c = {"workload": args.workload, "encoding": GEMM_ENC[args.workload], "shapes_out_in": GEMM_WORKLOADS[args.workload],
             "m": args.batch if args.batch > 1 else 512,
             "activation": "fp32 N(0,1), split into two f16 terms on the device inside the timed region" if GEMM_ENC[args.workload] == "Q5_K"
                           else "fp32 N(0,1), quantized to int8 per 256 on the device inside the timed region",
             "weights": "N(0,0.02) packed on device, seeded" if GEMM_ENC[args.workload] == "Q4_K" else "random valid blocks (random codes and scales, fixed f16 d), seeded, uploaded",
             "l2": "rotating distinct weights larger than 2x L2 per sweep"}
    elif args.workload in ATTN_WORKLOADS:
        h, hkv, d = ATTN_WORKLOADS[args.workload]
        c = {"workload": args.workload, "heads": h, "kv_heads": hkv, "head_dim": d, "batch": max(1, args.batch), "context": args.context,
             "kv": "f16 resident, N(0,1)", "l2": "rotating distinct caches larger than 2x L2 per sweep"}
    elif args.workload in MATVEC_WORKLOADS:
        enc, shapes, _, _ = MATVEC_WORKLOADS[args.workload]
        c = {"workload": args.workload, "encoding": enc, "shapes_out_in": shapes, "m": 1,
             "l2": "rotating distinct weights larger than 2x L2 per sweep", "activation": "fp32 N(0,1)",
             "weights": "N(0,0.02) packed on device, seeded" if enc in ("Q4_K", "Q8_0") else "random valid blocks (random codes and scales, fixed f16 d), seeded, uploaded"}
    else:
        model, ctx = DECODE_WORKLOADS[args.workload]
        cfg = model_config(model)
        c = {"workload": args.workload, "layers": cfg.n_layers, "d_model": cfg.d_model, "ffn": cfg.ffn_dim, "heads": cfg.n_heads,
             "kv_heads": cfg.n_kv_heads, "vocab": cfg.vocab, "linear": cfg.linear_enc, "tables": cfg.table_enc, "batch": args.batch,
             "context": ctx, "context_fill": "seeded noise K/V (no prompt pass)", "parallelism": f"tp{world}",
             "l2": "weights per step far larger than L2", "weights": "N(0,0.02) packed on device, seeded"}
        if args.workload in MIXED_WORKLOADS:
            c["linear"] = "Q4_K; attn_v and ffn_down of every second layer Q6_K"
            c["weights"] += "; the Q6_K tensors: random valid blocks (random codes and scales, f16 d = 6e-5), seeded, uploaded"
    if extra:
        c.update(extra)
    return c


# ---------------------------------------------------------------------------------------------------
# our arm: matvec sweep
# ---------------------------------------------------------------------------------------------------
def read_floor_ms(torch, L, weights_flat, stream, steps: int) -> float:
    """ms per sweep of a kernel that only reads the same weights (one launch per weight, one graph per sweep)."""
    lib = L.lib(); sp = stream.cuda_stream
    with torch.cuda.stream(stream):
        for w in weights_flat:
            L.check(lib.skainet_cuda_probe_read_dev(w.handle, sp))
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for w in weights_flat:
                L.check(lib.skainet_cuda_probe_read_dev(w.handle, sp))
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / steps


def matmul_launches(w) -> int:
    """Kernels one skainet_cuda_matmul_dev call of one activation row launches: a Q4_K weight of 4 MiB or more with at
    most 12288 columns takes the ring kernel with the quantizer in its prologue (one launch); everything else is a quantizer
    launch followed by the matvec (csrc/api.cu)."""
    if w.encoding == "Q5_K":                # fp32 activations: no quantizer
        return 1
    return 1 if (w.encoding == "Q4_K" and w.packed_bytes >= (4 << 20) and w.cols <= 12288) else 2


def matvec_sweep_rate(torch, device, L, weights_flat, stream, steps: int, warmup: int):
    """Times `steps` sweeps of one fused-path matvec per weight (fp32 activation in HBM), one CUDA graph
    per sweep, on `stream`. Returns (ms per sweep, launches per sweep)."""
    xs, ys = {}, {}
    gen = torch.Generator(device="cuda").manual_seed(5)
    for w in weights_flat:
        if w.cols not in xs:
            xs[w.cols] = torch.randn(w.cols, device="cuda", generator=gen, dtype=torch.float32)
        if w.rows not in ys:
            ys[w.rows] = torch.empty(w.rows, device="cuda", dtype=torch.float32)
    sp = stream.cuda_stream

    def sweep():
        for w in weights_flat:
            device.matmul(w, xs[w.cols].data_ptr(), 1, ys[w.rows].data_ptr(), L.ACT_NATIVE, sp)

    with torch.cuda.stream(stream):
        sweep(); stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            sweep()
        for _ in range(max(3, warmup)):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / steps, sum(matmul_launches(w) for w in weights_flat), graph, (xs, ys)


def matvec_configs_summary(torch, device, L, steps: int = 10) -> dict:
    """Benchmark configs 1 (Q8_0 4096x4096) and 2 (Q4_K 11008x4096 + 4096x11008) at M = 1, measured in the same process as the
    decode line: algorithmic GB/s of the whole matvec call (activation quantization included) over a rotation of distinct weights larger than 2x L2, the
    fraction of the measured copy bandwidth, and the time a kernel that only reads the same bytes takes."""
    info = device.device_info()
    peak, _ = load_peaks()
    out = {}
    stream = torch.cuda.Stream()
    for name, key in (("q8_0_matvec", "config1_q8_0_4096x4096"), ("q4k_matvec", "config2_q4k_11008x4096_4096x11008")):
        enc, shapes, bb, be = MATVEC_WORKLOADS[name]
        copies = max(2, int(np.ceil(2.2 * info["l2_bytes"] / min(r * (c // be) * bb for r, c in shapes))))
        ws = [device.Weight.synth(enc, r, c, seed=50 + 10 * si + ci, std=0.02) for ci in range(copies) for si, (r, c) in enumerate(shapes)]
        nbytes = sum(algorithmic_bytes(bb, be, w.rows, w.cols) for w in ws)
        ms, launches, graph, keep = matvec_sweep_rate(torch, device, L, ws, stream, steps, 3)
        floor = read_floor_ms(torch, L, ws, stream, steps)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[key] = {"gbs": gbs, "frac": gbs / peak, "avg_launch_us": ms * 1e3 / len(ws), "read_floor_us": floor * 1e3 / len(ws),
                    "weights": len(ws), "launches_per_matvec": launches / len(ws)}
        del graph, keep
        for w in ws:
            w.free()
    out["note"] = ("M = 1 through skainet_cuda_matmul_dev, one CUDA graph per sweep; config 1 = activation quantizer launch + matvec launch, config 2 = one "
                   "launch (the ring kernel quantizes the row in its prologue); avg_launch_us is per matvec; frac of the measured copy bandwidth")
    return out


def run_matvec(args) -> None:
    import torch
    import torch.distributed as dist
    from skainet_b200 import _lib as L, device
    rank, world, local = dist_env()
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local); device.set_device(local)
    info = device.device_info()
    enc, shapes, bb, be = MATVEC_WORKLOADS[args.workload]
    copies = max(2, int(np.ceil(2.2 * info["l2_bytes"] / min(r * (c // be) * bb for r, c in shapes))))
    if enc in ("Q4_K", "Q8_0"):
        weights = [device.Weight.synth(enc, r, c, seed=1000 * rank + 10 * si + ci, std=0.02) for ci in range(copies) for si, (r, c) in enumerate(shapes)]
    else:                                   # random valid blocks packed on the host (the reference's microbench fixture style)
        hrng = np.random.default_rng(1000 * rank + 3)
        weights = [device.Weight.upload(random_blocks(hrng, enc, r, c), enc, r, c) for ci in range(copies) for si, (r, c) in enumerate(shapes)]
    bytes_per_step = sum(algorithmic_bytes(bb, be, w.rows, w.cols) for w in weights)
    stream = torch.cuda.Stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    ms_step, launches, graph, bufs = matvec_sweep_rate(torch, device, L, weights, stream, args.steps, args.warmup)
    floor_ms = read_floor_ms(torch, L, weights, stream, args.steps)
    barrier()
    if rank == 0 and not args.skip_cpu:      # keep the GPU under load long enough for the clock sampler
        t_end = time.time() + 1.0
        with torch.cuda.stream(stream):
            while time.time() < t_end:
                graph.replay(); stream.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # end to end: host activation in, host output out, per matvec
    xs, ys = bufs
    hx = {c: torch.randn(c, dtype=torch.float32).pin_memory() for c in xs}
    hy = {r: torch.empty(r, dtype=torch.float32).pin_memory() for r in ys}
    lib = L.lib(); sp = stream.cuda_stream

    def e2e_sweep():
        for w in weights:
            L.check(lib.skainet_cuda_memcpy_h2d(xs[w.cols].data_ptr(), hx[w.cols].data_ptr(), w.cols * 4, sp))
            device.matmul(w, xs[w.cols].data_ptr(), 1, ys[w.rows].data_ptr(), L.ACT_NATIVE, sp)
            L.check(lib.skainet_cuda_memcpy_d2h(hy[w.rows].data_ptr(), ys[w.rows].data_ptr(), w.rows * 4, sp))   # synchronises

    e2e_steps = 0 if args.skip_e2e else max(1, min(args.steps, 5))
    e2e_ms = 0.0
    if e2e_steps:
        e2e_sweep(); barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(stream)
        for _ in range(e2e_steps):
            e2e_sweep()
        e3.record(stream); barrier()
        e2e_ms = e2.elapsed_time(e3)
    t = torch.tensor([ms_step, e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        peak, peak_kind = load_peaks()
        per_launch_us = ms_step * 1e3 / len(weights)
        achieved = bytes_per_step / (ms_step * 1e-3) / 1e9
        line = {
            "metric": f"{args.workload}_hbm_gbs", "value": achieved * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtype_of(args.workload), "data": "synthetic", "config": workload_config(args, world, {"weights_per_shape": copies}),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": bytes_per_step / len(weights) * {"Q4_K": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE, "Q8_0": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE, "Q6_K": 1.0003}[enc] if enc != "Q5_K" else None,
                         "traffic_source": {"Q4_K": "ncu dram bytes per launch of the 11008x4096 Q4_K capture, scaled by weight bytes",
                                            "Q8_0": "ncu dram bytes per launch of the 11008x4096 Q4_K capture, scaled by weight bytes",
                                            "Q6_K": "ncu dram bytes per q6k_rows_kernel launch on this workload's own shapes (36,998,400 and 37,005,568 read, 0 written, "
                                                    "against 36,986,880 of weights)", "Q5_K": None}[enc],
                         "peak_kind": peak_kind,
                         "kernel": {"Q4_K": "q4k_matvec_ring_kernel", "Q8_0": "q8_0_matvec_fused_kernel", "Q6_K": "q6k_rows_kernel", "Q5_K": "q5k_rows_kernel"}[enc],
                         "avg_launch_us": per_launch_us,
                         "read_floor_us": floor_ms * 1e3 / len(weights), "read_floor_gbs": bytes_per_step / (floor_ms * 1e-3) / 1e9,
                         "note": "avg launch = timed region / matvec calls; the activation quantizer (its own launch for Q8_0 and small weights, the "
                                 "matvec's prologue otherwise) and launch gaps are inside it. "
                                 "read_floor = a kernel that only reads the same weights, same launch count, same graph protocol"},
            "e2e": {"value": (bytes_per_step * world * e2e_steps / (e2e_ms * 1e-3) / 1e9) if e2e_steps else None, "unit": "GB/s",
                    "h2d_bytes_per_step": int(sum(4 * w.cols for w in weights)), "d2h_bytes_per_step": int(sum(4 * w.rows for w in weights)),
                    "note": "weights resident; each matvec copies its activation in and its output out and synchronises"},
            "gpu_launches": launches * args.steps, "clocks": clocks,
        }
        if world == 1 and not args.skip_cpu:
            cpu = cpu_matvec_rate(args.workload, 10.0)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------
# our arm: decode
# ---------------------------------------------------------------------------------------------------
def cpu_gemm_rate(workload: str, m: int, seconds: float) -> dict:
    """The reference has no batched kernel: its row-major Q4_K matvec is called once per activation row."""
    from oracle import ref as R
    shapes = GEMM_WORKLOADS[workload]
    enc = GEMM_ENC[workload]
    use_ref = R.ref() is not None
    rng = np.random.default_rng(5)
    items = [(r, c, random_blocks(rng, enc, r, c), rng.standard_normal(c).astype(np.float32)) for r, c in shapes]
    t0 = time.perf_counter(); calls = 0; flops = 0
    while time.perf_counter() - t0 < seconds:
        for r, c, packed, x in items:
            R.matmul(enc, x, packed, c, r, "rm", use_ref=use_ref); calls += 1; flops += 2 * r * c
    dt = time.perf_counter() - t0
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": 4 if use_ref else 1, "kind": "reference" if use_ref else "port",
            "sample": f"{calls} single-row calls of the reference's row-major {enc} kernel (it has no batched form); the rate per row "
                      f"does not depend on m = {m}", "seconds": dt}


def cpu_request_rate(workload: str, budget_s: float) -> dict:
    """The reference has no batched kernel, so a prompt token costs it one decode step: the request takes
    (prompt + generated) steps at the per-token rate of its composed decode step."""
    model, n_prompt, n_gen = REQUEST_WORKLOADS[workload]
    r = cpu_decode_rate(model, n_prompt, budget_s)
    return {"value": r["value"] * n_gen / (n_prompt + n_gen), "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"],
            "sample": f"generated tokens / ((prompt + generated) x per-token time); per-token time from: {r['sample']}", "seconds": r["seconds"]}


def run_request(args) -> None:
    """benchmark config 4 end to end: a 512-token prompt through the real prefill (batched-rows kernels, causal
    attention over the cache it fills), then 128 greedy tokens on the device. A step is one whole request;
    value = generated tokens / request time. The host-facing variant (`e2e`) sends the prompt from host memory
    and takes every generated token back through skainet_cuda_llama_decode."""
    import torch
    from skainet_b200 import device
    from skainet_b200.llama import Llama
    rank, world, local = dist_env()
    torch.cuda.set_device(local); device.set_device(local)
    model, n_prompt, n_gen = REQUEST_WORKLOADS[args.workload]
    cfg = model_config(model, max_seq=n_prompt + n_gen + 64, max_batch=1)
    m = Llama(cfg)
    m.synth(seed=100, std=0.02)
    m.finalize()
    prompt = (np.random.default_rng(11).integers(0, cfg.vocab, n_prompt)).astype(np.int32)
    mstream = torch.cuda.ExternalStream(m.stream)

    def request():
        m.reset()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record(mstream)
        nxt = m.prefill(prompt, seq=0)
        e[1].record(mstream)
        toks = m.generate(np.array([nxt], np.int32), n_gen - 1)
        e[2].record(mstream)
        torch.cuda.synchronize()
        return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), [nxt] + [int(t) for t in toks[:, 0]]

    warm = max(3, args.warmup)
    for _ in range(warm):
        request()
    sampler = ClockSampler(local); sampler.start()
    steps = max(1, min(args.steps, 16))
    pre, dec, toks = [], [], None
    for _ in range(steps):
        a, b, toks = request()
        pre.append(a); dec.append(b)
    clocks = sampler.stop()
    pre_ms, dec_ms = float(np.mean(pre)), float(np.mean(dec))
    # host-facing: prompt from host memory (it already is), every token back through the per-step call
    tin = torch.zeros(1, dtype=torch.int32).pin_memory(); tout = torch.zeros(1, dtype=torch.int32).pin_memory()
    m.reset()
    t0 = time.perf_counter()
    tin[0] = m.prefill(prompt, seq=0)
    for _ in range(n_gen - 1):
        m.decode_ptr(1, tin.data_ptr(), tout.data_ptr()); tin.copy_(tout)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    bytes_step, launches_step = m.step_cost(1)
    peak, peak_kind = load_peaks()
    dec_gbs = bytes_step * (n_gen - 1) / (dec_ms * 1e-3) / 1e9
    ms = pre_ms + dec_ms
    line = {"metric": "request_generated_tokens_per_s", "value": n_gen / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
            "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": dtype_of("decode_7b"), "data": "synthetic", "config": workload_config(args, 1),
            "phases": {"prefill_ms": pre_ms, "prefill_tokens_per_s": n_prompt / (pre_ms * 1e-3), "decode_ms": dec_ms,
                       "decode_tokens_per_s": (n_gen - 1) / (dec_ms * 1e-3)},
            "roofline": {"bound": "hbm", "achieved": dec_gbs, "peak": peak, "unit": "GB/s", "frac": dec_gbs / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "q4k_matvec_ring_kernel",
                         "note": "decode phase: bytes a step must read x steps / decode time (the prefill phase is tensor-bound: see the q4k_gemm workload)"},
            "e2e": {"value": n_gen / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 4 * n_prompt + 4 * (n_gen - 1),
                    "d2h_bytes_per_step": 4 * n_gen},
            "gpu_launches": launches_step * (n_gen - 1) * steps, "clocks": clocks, "tokens_head": toks[:4]}
    if not args.skip_cpu:
        cpu = cpu_request_rate(args.workload, 20.0)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    m.free()


def run_gemm(args) -> None:
    """m activation rows x Q4_K weights through skainet_cuda_matmul_dev: quantizer + tensor-core tile kernel.
    Operations = 2 * m * rows * cols per weight."""
    import torch
    from skainet_b200 import _lib as L, device
    rank, world, local = dist_env()
    torch.cuda.set_device(local); device.set_device(local)
    info = device.device_info()
    shapes = GEMM_WORKLOADS[args.workload]
    m = args.batch if args.batch > 1 else 512
    enc = GEMM_ENC[args.workload]
    copies = max(2, int(np.ceil(2.2 * info["l2_bytes"] / min(r * (c // 256) * BLOCK[enc][0] for r, c in shapes))) // 2)
    if enc == "Q4_K":
        ws = [device.Weight.synth("Q4_K", r, c, seed=10 * si + ci, std=0.02) for ci in range(copies) for si, (r, c) in enumerate(shapes)]
    else:
        hrng = np.random.default_rng(11)
        ws = [device.Weight.upload(random_blocks(hrng, enc, r, c), enc, r, c) for ci in range(copies) for si, (r, c) in enumerate(shapes)]
    gen = torch.Generator(device="cuda").manual_seed(3)
    xs = {c: torch.randn(m, c, device="cuda", generator=gen) for _, c in shapes}
    ys = {r: torch.empty(m, r, device="cuda") for r, _ in shapes}
    stream = torch.cuda.Stream(); sp = stream.cuda_stream
    ops = sum(2 * m * w.rows * w.cols for w in ws)

    def sweep():
        for w in ws:
            device.matmul(w, xs[w.cols].data_ptr(), m, ys[w.rows].data_ptr(), L.ACT_NATIVE, sp)

    warm = max(3, args.warmup)
    with torch.cuda.stream(stream):
        for _ in range(warm):
            sweep()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clk = ClockSampler(local); clk.start()
        stream.synchronize(); e0.record(stream)
        for _ in range(args.steps):
            sweep()
        e1.record(stream); stream.synchronize()
        clocks = clk.stop()
    ms_step = e0.elapsed_time(e1) / args.steps
    e2e_ms = None
    if not args.skip_e2e:                     # activations from pinned host memory, results back, per call
        hx = {c: torch.randn(m, c).pin_memory() for _, c in shapes}
        hy = {r: torch.empty(m, r).pin_memory() for r, _ in shapes}
        with torch.cuda.stream(stream):
            def e2e_sweep():
                for w in ws:
                    xs[w.cols].copy_(hx[w.cols], non_blocking=True)
                    device.matmul(w, xs[w.cols].data_ptr(), m, ys[w.rows].data_ptr(), L.ACT_NATIVE, sp)
                    hy[w.rows].copy_(ys[w.rows], non_blocking=True); stream.synchronize()
            e2e_sweep()
            t0 = time.perf_counter(); e2e_sweep(); e2e_ms = (time.perf_counter() - t0) * 1e3
    peak, peak_kind = load_tensor_peak()
    achieved = ops / (ms_step * 1e-3) / 1e12
    if enc == "Q4_K":
        kernel = "q4k_gemm_tc_kernel" if m >= 288 else "q4k_gemm_mma_kernel"
    elif enc == "Q6_K":
        kernel = "q6k_gemm_mma_kernel" if m >= 9 else "q6k_rows_kernel"
    else:
        kernel = "q5k_gemm_mma_kernel" if m >= 5 else "q5k_rows_kernel"
    line = {"metric": f"{args.workload}_tflops", "value": achieved, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_of(args.workload),
            "data": "synthetic", "config": workload_config(args, 1, {"weights_per_shape": copies}),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                         "peak_kind": peak_kind, "kernel": kernel, "avg_launch_us": ms_step * 1e3 / len(ws),
                         "note": "integer multiply-adds counted as 2 operations each; avg launch = timed region / calls (quantizer inside)"},
            "e2e": {"value": (ops / (e2e_ms * 1e-3) / 1e12) if e2e_ms else None, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": int(sum(4 * m * w.cols for w in ws)), "d2h_bytes_per_step": int(sum(4 * m * w.rows for w in ws))},
            "gpu_launches": 2 * len(ws) * args.steps, "clocks": clocks}
    if not args.skip_cpu:
        cpu = cpu_gemm_rate(args.workload, m, 10.0)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)


def run_attn(args) -> None:
    """Decode attention alone through skainet_cuda_attn_decode_dev: one query row per head against a
    resident f16 cache. Bytes per call = the K and V rows it must read."""
    import torch
    from skainet_b200 import _lib as L, device
    rank, world, local = dist_env()
    torch.cuda.set_device(local); device.set_device(local)
    info = device.device_info()
    h, hkv, d = ATTN_WORKLOADS[args.workload]
    batch, ctx = max(1, args.batch), args.context
    stride = ctx + 64
    call_bytes = 2 * batch * hkv * ctx * d * 2
    copies = int(min(max(2, np.ceil(2.2 * info["l2_bytes"] / call_bytes)), max(2, (4 << 30) // (2 * batch * hkv * stride * d * 2))))
    gen = torch.Generator(device="cuda").manual_seed(7 + rank)
    ks = [torch.randn(batch, hkv, stride, d, device="cuda", generator=gen).half() for _ in range(copies)]
    vs = [torch.randn(batch, hkv, stride, d, device="cuda", generator=gen).half() for _ in range(copies)]
    q = torch.randn(batch, h * d, device="cuda", generator=gen)
    out = torch.empty(batch, h * d, device="cuda")
    lens = torch.full((batch,), ctx, device="cuda", dtype=torch.int32)
    stream = torch.cuda.Stream(); sp = stream.cuda_stream

    def sweep():
        for k, v in zip(ks, vs):
            device.attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), batch, h, hkv, d, stride, lens.data_ptr(), ctx,
                               d ** -0.5, 0, sp)

    warm = max(3, args.warmup)
    with torch.cuda.stream(stream):
        sweep(); stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            sweep()
        for _ in range(warm):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clk = ClockSampler(local); clk.start()
        stream.synchronize(); e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream); stream.synchronize()
        clocks = clk.stop()
    ms_step = e0.elapsed_time(e1) / args.steps
    # end to end: q from pinned host memory, result back, per call
    hq = torch.randn(batch, h * d).pin_memory(); hout = torch.empty(batch, h * d).pin_memory()
    e2e_ms = None
    if not args.skip_e2e:
        with torch.cuda.stream(stream):
            def e2e_sweep():
                for k, v in zip(ks, vs):
                    q.copy_(hq, non_blocking=True)
                    device.attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), batch, h, hkv, d, stride, lens.data_ptr(),
                                       ctx, d ** -0.5, 0, sp)
                    hout.copy_(out, non_blocking=True); stream.synchronize()
            e2e_sweep()
            t0 = time.perf_counter(); e2e_sweep(); e2e_ms = (time.perf_counter() - t0) * 1e3
    peak, peak_kind = load_peaks()
    achieved = call_bytes * copies / (ms_step * 1e-3) / 1e9
    line = {"metric": "attn_decode_hbm_gbs", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 K/V, f32 q split in two f16 terms, f32 accumulate", "data": "synthetic",
            "config": workload_config(args, 1, {"caches": copies}),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_kind": peak_kind, "kernel": "attn_decode_mma_kernel", "avg_launch_us": ms_step * 1e3 / copies,
                         "note": "avg launch = timed region / calls; each call is the split-K kernel plus its merge"},
            "e2e": {"value": (call_bytes * copies / (e2e_ms * 1e-3) / 1e9) if e2e_ms else None, "unit": "GB/s",
                    "h2d_bytes_per_step": 4 * batch * h * d * copies, "d2h_bytes_per_step": 4 * batch * h * d * copies},
            "gpu_launches": 2 * copies * args.steps, "clocks": clocks}
    if not args.skip_cpu:
        cpu = cpu_attn_rate(args.workload, ctx, batch)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)


def tp_parity_check(torch, dist, m, cfg, model_name: str, ctx: int, batch: int, rank: int, world: int, n_steps: int = 4) -> dict:
    """Correctness of the tensor-parallel run against the single-GPU model, inside the bench: rank 0 also builds the
    unsharded model of the same seed (it fits beside its shard), both decode the same seeded context with the same
    teacher tokens for a few steps, and the logits are compared.

    What "agree" can mean here is measured, not assumed. Every int8 activation quantizer on the path turns a relative
    input difference e into about 0.15 * sqrt(e) at its output, so two correct implementations that differ in fp32
    summation order (as a sharded sum must) settle percents apart after 80 layers. The yardstick is therefore a
    control: the unsharded model run twice on rank 0 through different kernels (one activation row: the streaming
    matvecs; the same row as the first of two: the tile kernels). `within_control` says the sharded run is no further
    from the single-GPU run than a few times that; the 2e-3 bar of the 2-layer parity test is reported as `within_bar`.
    Only a gross error (beyond both 5e-2 and four times the control: a wrong shard, a lost partial sum) fails the run."""
    from skainet_b200.llama import Llama
    first = (np.arange(1, batch + 1, dtype=np.int32) * 17 % cfg.vocab).astype(np.int32)
    ref = None
    ref_logits, ref_tokens, margins, control = [], [], [], []
    if rank == 0:
        ref = Llama(model_config(model_name, max_seq=cfg.max_seq, max_batch=max(batch, 2), tp_rank=0, tp_world=1))
        ref.synth(seed=100, std=0.02)
        ref.finalize()
        for b in range(batch):
            ref.fake_prefill(ctx, seq=b, seed=7 + b)
        tin, tout = first.copy(), np.zeros(batch, np.int32)
        for _ in range(n_steps):                              # the single-GPU run: its greedy tokens are the teacher
            ref_tokens.append(tin.copy())
            ref.decode(tin, tout)
            lg = ref.logits(batch).copy()
            ref_logits.append(lg)
            srt = np.sort(lg, axis=1)
            margins.append(float(((srt[:, -1] - srt[:, -2]) / np.sqrt(np.mean(lg.astype(np.float64) ** 2))).min()))
            tin = tout.copy()
        if batch == 1:                                        # control: the same row as the first of two identical sequences
            ref.reset()
            ref.fake_prefill(ctx, seq=0, seed=7)
            ref.fake_prefill(ctx, seq=1, seed=(7 - 31) % (1 << 64))      # the per-sequence seed offset cancels: same noise as sequence 0
            t2, o2 = np.zeros(2, np.int32), np.zeros(2, np.int32)
            for i in range(n_steps):
                t2[:] = ref_tokens[i][0]
                ref.decode(t2, o2)
                lg2 = ref.logits(2)[0].astype(np.float64)
                a = ref_logits[i][0].astype(np.float64)
                control.append(float(np.abs(lg2 - a).max() / np.sqrt(np.mean(a * a))))
        ref.free()
    m.reset()
    for b in range(batch):
        m.fake_prefill(ctx, seq=b, seed=7 + b)
    errs, equal = [], True
    tin, tout = np.zeros(batch, np.int32), np.zeros(batch, np.int32)
    tok = torch.zeros(batch, dtype=torch.int32, device="cuda")
    for i in range(n_steps):
        if rank == 0:
            tok = torch.from_numpy(ref_tokens[i].copy()).cuda()
        dist.broadcast(tok, src=0)                             # teacher tokens: the single-GPU model's greedy choice
        tin[:] = tok.cpu().numpy()
        m.decode(tin, tout)
        lg_tp = m.logits(batch)                                # all ranks take part in the gather
        if rank == 0:
            a = ref_logits[i].astype(np.float64)
            errs.append(float(np.abs(lg_tp.astype(np.float64) - a).max() / np.sqrt(np.mean(a * a))))
            nxt = ref_tokens[i + 1] if i + 1 < n_steps else None
            if nxt is not None:
                equal = equal and bool(np.array_equal(tout, nxt))
    out, ok = None, True
    if rank == 0:
        worst, ctl = max(errs), (max(control) if control else None)
        ok = worst <= max(5e-2, 4.0 * (ctl or 0.0))
        out = {"steps": n_steps, "max_rel_logit_err": worst, "per_step": errs, "tokens_equal": equal, "min_top2_margin": min(margins),
               "control_rel_logit_err": ctl, "control": "the unsharded model on rank 0 through its one-row kernels against the same row through its tile kernels",
               "within_control": (worst <= 4.0 * ctl) if ctl else None, "bar": 2e-3, "within_bar": worst <= 2e-3,
               "reference": "the unsharded model of the same seed on rank 0, same seeded context, teacher-forced"}
    flag = torch.tensor([1 if ok else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag[0]) != 1:
        raise SystemExit(f"tensor-parallel logits differ grossly from the single-GPU model: {out}")
    # back to the state the timed region starts from
    m.reset()
    for b in range(batch):
        m.fake_prefill(ctx, seq=b, seed=7 + b)
    return out


def run_kv_turboquant(args) -> None:
    """kv_turboquant: the TurboQuant KV store (4-bit keys and values, 8 heads x 128) behind one decode step of attention over
    --context positions: decode of the window's blocks to fp32 + fp32 attention, per layer of a 32-layer store (the layers'
    blocks together exceed L2). Also times the append (encode) of one token."""
    import torch
    from skainet_b200 import _lib as L, device
    from skainet_b200.kvstore import DeviceKvCacheStore, TurboQuantConfig
    rank, world, local = dist_env()
    torch.cuda.set_device(local); device.set_device(local)
    layers, heads, d, ctx = 32, 8, 128, args.context
    st = DeviceKvCacheStore(layers, heads, d, ctx + 8, keyConfig=TurboQuantConfig.polarOnly(4), valueConfig=TurboQuantConfig.polarOnly(4))
    gen = torch.Generator(device="cuda").manual_seed(3)
    kv = torch.randn(2, heads * d, device="cuda", generator=gen)
    stream = torch.cuda.Stream(); sp = stream.cuda_stream
    with torch.cuda.stream(stream):
        for _ in range(ctx):
            for l in range(layers):
                st.appendTokenDevice(l, kv[0].data_ptr(), kv[1].data_ptr(), sp)
        stream.synchronize()
        q = torch.randn(heads * d, device="cuda", generator=gen); out = torch.empty(heads * d, device="cuda")

        def sweep():
            for l in range(layers):
                st.decodeStep(l, q.data_ptr(), out.data_ptr(), heads, 0, ctx, 0.0, sp)
        sweep(); stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            sweep()
        warm = max(3, args.warmup)
        for _ in range(warm):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clk = ClockSampler(local); clk.start()
        stream.synchronize(); e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream); stream.synchronize()
        clocks = clk.stop()
        ms_step = e0.elapsed_time(e1) / args.steps
        # append (encode) of one more token into every layer
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(stream)
        for l in range(layers):
            st.appendTokenDevice(l, kv[0].data_ptr(), kv[1].data_ptr(), sp)
        e3.record(stream); stream.synchronize()
        append_us = e2.elapsed_time(e3) * 1e3 / layers
    block = 64 + 16 + 4                               # 4-bit codes + four fp32 scales + the seed word the reference counts
    call_bytes = 2 * heads * ctx * (64 + 16)          # compressed bytes one call must read
    window_bytes = 2 * heads * ctx * d * 4            # the fp32 window written by the decode and read by the attention
    peak, peak_kind = load_peaks()
    us = ms_step * 1e3 / layers
    achieved = (call_bytes + 2 * window_bytes) / (us * 1e-6) / 1e9
    status = L.lib().skainet_cuda_device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: {L.last_error()}")
    line = {"metric": "kv_turboquant_attn_us", "value": us, "unit": "us", "n_gpus": 1, "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "4-bit codes + fp32 scales -> fp32", "data": "synthetic",
            "config": {"workload": "kv_turboquant", "layers": layers, "heads": heads, "head_dim": d, "context": ctx, "key_bits": 4, "value_bits": 4,
                       "block_bytes": block, "l2": f"{layers} layers x {call_bytes / 1e6:.1f} MB of blocks rotate"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                         "kernel": "tq_decode_kernel", "note": "bytes = compressed blocks read + the fp32 window written once and read once; a first "
                                                               "version: the blocks are decoded to fp32 rows and attended by the fp32 kernel",
                         "compressed_bytes_per_call": call_bytes, "fp32_window_bytes": window_bytes},
            "append_us_per_layer": append_us, "gpu_launches": 3 * layers * args.steps, "clocks": clocks,
            "e2e": {"value": None, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "note": "device-resident entry points only"}}
    print(json.dumps(line), flush=True)
    st.free()


def tp_exchange_times(m, torch, dist, rounds: int = 64, reps: int = 20) -> dict:
    """The group exchanges of a decode step timed on their own (every rank calls; the max over ranks is reported):
    device microseconds per exchange of one [d_model] fp32 row, `rounds` launches back to back in one CUDA graph."""
    out = {}
    for key, mode in (("peer_sum_us", 0), ("send_gather_norm_quant_us", 1), ("nccl_sum_us", 2)):
        t = torch.tensor([m.tp_exchange_time(mode, rounds, reps)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[key] = float(t[0])
    out["note"] = (f"{rounds} exchanges of one [d_model] fp32 row per CUDA graph, {reps} replays between two events, max over ranks. peer_sum: in-place "
                   "sum through peer memory; send_gather_norm_quant: store + gather + sum + RMSNorm + quantize in one kernel (the decode step's "
                   "matvec epilogue does the store part itself); nccl_sum: ncclAllReduce of the same row")
    return out


def run_collective(args) -> None:
    """tp_collective: nothing but the exchanges, on a one-layer model of the 70B width."""
    import torch
    import torch.distributed as dist
    from skainet_b200 import _lib as L, device
    from skainet_b200.llama import Llama, LlamaConfig
    rank, world, local = dist_env()
    if world < 2:
        raise SystemExit("tp_collective needs 2 or more ranks (launch under torch.distributed.run with --gpus N)")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local); device.set_device(local)
    cfg = LlamaConfig(1, 8192, 64, 8, 128, 2048 * world, 256 * world, table_enc="Q4_K", max_seq=512, max_batch=1, tp_rank=rank, tp_world=world)
    m = Llama(cfg)
    m.synth(seed=3, std=0.02); m.finalize()
    ids = [Llama.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    m.tp_init(ids[0])
    sampler = ClockSampler(local)
    dist.barrier(); torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        m.tp_exchange_time(1, 8, 1)
    times = tp_exchange_times(m, torch, dist, rounds=64, reps=max(1, args.steps))
    clocks = sampler.stop() if rank == 0 else None
    status = L.lib().skainet_cuda_device_status()
    ok = torch.tensor([1 if status == 0 else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok[0]) != 1:
        raise SystemExit(f"rank {rank}: device status {status} ({L.last_error() if status else 'ok'})")
    if rank == 0:
        us = times["send_gather_norm_quant_us"]
        nbytes = 4 * cfg.d_model * (world - 1)          # what one rank stores into its peers per exchange
        print(json.dumps({
            "metric": "tp_exchange_us", "value": us, "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": us * 64 * 1e-3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": "tp_collective", "d_model": cfg.d_model, "row_bytes": 4 * cfg.d_model,
                                            "parallelism": f"tp{world}", "l2": "32 KB rows: latency, not bandwidth, is measured"},
            "tp_exchange": times,
            "roofline": {"bound": "nvlink", "achieved": nbytes / (us * 1e-6) / 1e9, "peak": 770.0, "unit": "GB/s", "frac": nbytes / (us * 1e-6) / 1e9 / 770.0,
                         "traffic": None, "note": "bytes one rank stores to its peers per exchange / time; a 32 KB exchange is bound by one NVLink store latency"},
            "gpu_launches": 64 * max(1, args.steps) * 3, "clocks": clocks}), flush=True)
    m.free()
    dist.destroy_process_group()


def run_decode(args) -> None:
    import torch
    import torch.distributed as dist
    from skainet_b200 import _lib as L, device
    from skainet_b200.llama import Llama, W_HEAD, W_O, W_DOWN, W_QKV, W_GATE_UP, W_Q, W_K, W_V
    rank, world, local = dist_env()
    mixed = args.workload in MIXED_WORKLOADS
    if mixed and world > 1:
        raise SystemExit(f"{args.workload} is a one-GPU workload")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local); device.set_device(local)
    model_name, ctx = DECODE_WORKLOADS[args.workload]
    batch = args.batch
    cfg = model_config(model_name, max_seq=ctx + 2048, max_batch=batch, tp_rank=rank, tp_world=world)
    m = Llama(cfg)
    m.synth(seed=100, std=0.02)
    mixed_layers = list(range(0, cfg.n_layers, 2)) if mixed else []
    if mixed:
        hrng = np.random.default_rng(17)
        for l in mixed_layers:
            for which, rows, cols in ((W_V, cfg.n_kv_heads * cfg.head_dim, cfg.d_model), (W_DOWN, cfg.d_model, cfg.ffn_dim)):
                packed = random_blocks(hrng, "Q6_K", rows, cols)
                packed.reshape(-1, 210)[:, 208:210] = np.array([6e-5], np.float16).view(np.uint8)
                m.set_weight(l, which, device.Weight.upload(packed, "Q6_K", rows, cols))
    m.finalize()
    if world > 1:
        ids = [Llama.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        m.tp_init(ids[0])
    for b in range(batch):
        m.fake_prefill(ctx, seq=b, seed=7 + b)
    first = np.arange(1, batch + 1, dtype=np.int32) * 17 % cfg.vocab
    mstream = torch.cuda.ExternalStream(m.stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(3, args.warmup)
    barrier()                                             # ranks start their first step together (peer waits are bounded)
    m.generate(first, warm)
    bytes_step, launches_step = m.step_cost(batch)
    tp_parity = tp_parity_check(torch, dist, m, cfg, model_name, ctx, batch, rank, world) if world > 1 else None
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()

    def block():                                          # EXACTLY `steps` decode steps, device-timed on the model's stream
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(mstream)
        t = m.generate(first, args.steps)                 # K graph replays, synchronises at the end
        e1.record(mstream)
        barrier()
        return e0.elapsed_time(e1), t

    # The block is repeated until about a second has been timed (a single block of 20 steps is 0.1-0.2 s, too short to
    # be stable); every rank runs the same number of blocks, and the median block is reported.
    ms0, toks = block()
    tm = torch.tensor([ms0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    room = max(0, (cfg.max_seq - ctx - warm - 200) // max(1, args.steps) - 1)       # decode positions left in the cache
    extra = int(min(15, room, max(0, np.ceil(1000.0 / max(float(tm[0]), 1e-3)) - 1)))
    block_ms = [ms0] + [block()[0] for _ in range(extra)]
    ms = float(np.median(block_ms))
    clocks = sampler.stop() if rank == 0 else None
    logits_ok = bool(np.isfinite(m.logits(batch)).all())
    tokens_ok = bool(((toks >= 0) & (toks < cfg.vocab)).all())

    # end to end: one C-ABI call per step, token ids from pinned host memory and back
    e2e_steps = 0 if args.skip_e2e else max(1, min(args.steps, 64))
    e2e_ms = 0.0
    if e2e_steps:
        tin = torch.from_numpy(first.copy()).pin_memory(); tout = torch.zeros(batch, dtype=torch.int32).pin_memory()
        for _ in range(2):
            m.decode_ptr(batch, tin.data_ptr(), tout.data_ptr()); tin.copy_(tout)
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(mstream)
        for _ in range(e2e_steps):
            m.decode_ptr(batch, tin.data_ptr(), tout.data_ptr()); tin.copy_(tout)
        e3.record(mstream); barrier()
        e2e_ms = e2.elapsed_time(e3)

    # the matvec kernel alone over this rank's own weights (every layer's four linears + the head)
    ws = []
    for l in range(cfg.n_layers):
        qkv = [m.weight(l, W_Q), m.weight(l, W_K), m.weight(l, W_V)] if l in mixed_layers else [m.weight(l, W_QKV)]     # a Q6_K attn_v is not merged
        ws += qkv + [m.weight(l, W_O), m.weight(l, W_GATE_UP), m.weight(l, W_DOWN)]
    ws.append(m.weight(0, W_HEAD))
    mv_bytes = sum(algorithmic_bytes(*BLOCK[w.encoding], w.rows, w.cols) for w in ws)
    stream = torch.cuda.Stream()
    mv_ms, _, _, _ = matvec_sweep_rate(torch, device, L, ws, stream, max(2, min(args.steps, 10)), 3)

    t = torch.tensor([ms, e2e_ms, mv_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, mv_ms = float(t[0]), float(t[1]), float(t[2])
    # a run in which a bounded device wait gave up, or whose outputs are not numbers, must not print a number
    status = L.lib().skainet_cuda_device_status()
    ok = torch.tensor([1 if (status == 0 and logits_ok and tokens_ok) else 0], device="cuda", dtype=torch.int32)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok[0]) != 1:
        raise SystemExit(f"rank {rank}: device status {status} ({L.last_error() if status else 'ok'}), logits finite {logits_ok}, tokens in range {tokens_ok}")
    matvec_summary = matvec_configs_summary(torch, device, L) if (world == 1 and not args.skip_cpu) else None
    tp_exchange = tp_exchange_times(m, torch, dist) if (world > 1 and batch == 1) else None
    if rank == 0:
        peak, peak_kind = load_peaks()
        achieved = mv_bytes / (mv_ms * 1e-3) / 1e9
        step_gbs = bytes_step / (ms / args.steps * 1e-3) / 1e9
        # the bytes one launch of the dominant kernel must move (its own weight), and the DRAM bytes ncu counted for it
        launch_bytes = mv_bytes / len(ws)
        line = {
            "metric": "decode_tokens_per_s", "value": batch * args.steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": dtype_of(args.workload), "data": "synthetic", "config": workload_config(args, world),
            "roofline": {"bound": "hbm", "achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak,
                         "traffic": launch_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                         "traffic_source": "dram read+write bytes of one q4k_matvec_ring_kernel launch from the ncu captures summarised in "
                                           "profiles/ (1.001 x the weight bytes at 25 MB and at 264 MB), scaled to this run's mean weight size",
                         "peak_kind": peak_kind, "kernel": "q4k_matvec_ring_kernel" + (" (Q6_K tensors: q6k_rows_kernel)" if mixed else ""),
                         "note": "per GPU. achieved / frac: bytes one decode step must read (weights once + visible K/V) / measured step time. "
                                 "kernel_*: the matvec path alone (quantizer + matvec) swept over this rank's own weights in a CUDA graph",
                         "step_bytes_per_gpu": bytes_step, "kernel_achieved": achieved, "kernel_frac": achieved / peak,
                         "kernel_avg_launch_us": mv_ms * 1e3 / len(ws)},
            "timing": {"blocks": len(block_ms), "block_ms_min": float(min(block_ms)), "block_ms_median": ms, "block_ms_max": float(max(block_ms)),
                       "note": "each block = exactly `steps` steps between barriers, CUDA events on the model's stream; the median block is reported"},
            "e2e": {"value": (batch * e2e_steps / (e2e_ms * 1e-3)) if e2e_steps else None, "unit": "tokens/s",
                    "h2d_bytes_per_step": 4 * batch, "d2h_bytes_per_step": 4 * batch,
                    "note": "one skainet_cuda_llama_decode call per step: pinned host token ids in, arg-max ids out, host sync each step"},
            "gpu_launches": launches_step * args.steps, "clocks": clocks, "tokens_head": [int(x) for x in toks[:4, 0]],
            "checks": {"device_status": 0, "logits_finite": True, "tokens_in_vocab": True},
        }
        if tp_parity is not None:
            line["tp_parity"] = tp_parity
        if tp_exchange is not None:
            line["tp_exchange"] = tp_exchange
        if matvec_summary is not None:
            line["matvec"] = matvec_summary
        if world == 1 and not args.skip_cpu:
            cpu = cpu_decode_rate(model_name, ctx, 20.0, mixed=mixed)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    m.free()
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="decode_70b", choices=sorted(MATVEC_WORKLOADS) + sorted(DECODE_WORKLOADS) + sorted(ATTN_WORKLOADS) + sorted(GEMM_WORKLOADS) + sorted(REQUEST_WORKLOADS) + ["tp_collective", "kv_turboquant"])
    ap.add_argument("--context", type=int, default=4096, help="keys per sequence (attn_decode workload)")
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded together (decode workloads)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in MATVEC_WORKLOADS:
        run_matvec(args)
    elif args.workload in ATTN_WORKLOADS:
        run_attn(args)
    elif args.workload in GEMM_WORKLOADS:
        run_gemm(args)
    elif args.workload in REQUEST_WORKLOADS:
        run_request(args)
    elif args.workload == "tp_collective":
        run_collective(args)
    elif args.workload == "kv_turboquant":
        run_kv_turboquant(args)
    else:
        run_decode(args)


if __name__ == "__main__":
    main()
