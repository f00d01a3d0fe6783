#!/usr/bin/env python
"""Benchmark of the packed-quantized decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0). Workloads:

  q4k_matvec (default) — BASELINE config 2 at M=1: Q4_K dequant-fused matvec over W[11008,4096] and
      W[4096,11008] (seeded N(0,0.02) weights packed on the device), fp32 activations ~N(0,1).
      A step is one sweep over 2 x COPIES distinct weights (> 2x L2, so HBM serves every byte).
      metric = algorithmic HBM GB/s (weight bytes + activation + output per matvec).
  q8_0_matvec — BASELINE config 1: Q8_0 W[4096,4096], same protocol.

`value` is timed with the inputs resident in HBM, the sweep captured in one CUDA graph; `e2e` is the
same sweep driven through the C ABI with HOST activations and outputs (pinned), host<->device copies
inside the timed region, weights resident (uploaded once at load, as a SKaiNET provider does).
`--impl reference` times the reference's own C kernels (oracle/_ref, else the port) on the host.
PyTorch is used here for streams, events, pinned memory and the process group only.
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

WORKLOADS = {
    # name: (encoding, [(rows=out, cols=in), ...], block bytes, block elems)
    "q4k_matvec": ("Q4_K", [(11008, 4096), (4096, 11008)], 144, 256),
    "q8_0_matvec": ("Q8_0", [(4096, 4096)], 34, 32),
}


def algorithmic_bytes(enc_bytes: int, enc_elems: int, rows: int, cols: int, m: int = 1) -> int:
    """Bytes one matvec must move: packed weight once, activation in, output out (fp32)."""
    return rows * (cols // enc_elems) * enc_bytes + 4 * m * (rows + cols)


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
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ---------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own C kernels on the host cores
# ---------------------------------------------------------------------------------------------------
def cpu_matvec_rate(workload: str, seconds: float, rng_seed: int = 5) -> dict:
    """Times the reference's compiled C matvec (oracle/_ref; the port if it is absent) on this host for
    about `seconds`, on the workload's shapes with one weight per shape. Returns GB/s of algorithmic bytes."""
    from oracle import ref as R
    enc, shapes, bb, be = WORKLOADS[workload]
    use_ref = R.ref() is not None
    rng = np.random.default_rng(rng_seed)
    items = []
    for rows, cols in shapes:
        packed = rng.integers(0, 256, size=rows * (cols // be) * bb, dtype=np.uint8)
        blk = packed.reshape(-1, bb)
        blk[:, 0:2] = np.array([0.01], np.float16).view(np.uint8)       # sane f16 scale fields
        if enc == "Q4_K":
            blk[:, 2:4] = np.array([0.01], np.float16).view(np.uint8)
        items.append((rows, cols, packed, rng.standard_normal(cols).astype(np.float32)))
    for rows, cols, packed, x in items:                                     # warm-up (spins the row pool up)
        R.matmul(enc, x, packed, cols, rows, "rm", use_ref=use_ref)
    t0 = time.perf_counter(); done = 0; calls = 0
    while time.perf_counter() - t0 < seconds:
        for rows, cols, packed, x in items:
            R.matmul(enc, x, packed, cols, rows, "rm", use_ref=use_ref)
            done += algorithmic_bytes(bb, be, rows, cols); calls += 1
    dt = time.perf_counter() - t0
    return {"value": done / dt / 1e9, "unit": "GB/s", "cores": 4 if use_ref else 1, "kind": "reference" if use_ref else "port",
            "sample": f"{calls} matvec calls over the workload's {len(items)} shapes in {dt:.1f} s, "
                      f"{'skainet_%s_matmul_rm (reference C, its 4-thread row pool)' % ('q4k' if enc == 'Q4_K' else 'q8_0') if use_ref else 'oracle port, scalar'}"
                      f" of {os.cpu_count()} host cores", "calls": calls, "seconds": dt}


def run_reference(args) -> None:
    rank, world, _ = dist_env()
    if rank != 0:
        return
    enc, shapes, bb, be = WORKLOADS[args.workload]
    per_step = max(1.0, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    cpu_matvec_rate(args.workload, 0.5)
    times, vals = [], []
    for i in range(args.warmup + args.steps):
        r = cpu_matvec_rate(args.workload, per_step)
        if i >= args.warmup:
            times.append(r["seconds"] * 1e3); vals.append(r["value"])
    r["value"] = float(np.mean(vals))
    line = {"impl": "reference", "metric": f"{args.workload}_hbm_gbs", "value": r["value"], "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times)), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4 -> int32, f32 accumulate" if enc == "Q4_K" else "f32",
            "data": "synthetic", "config": workload_config(args.workload, 1),
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(workload: str, copies: int) -> dict:
    enc, shapes, bb, be = WORKLOADS[workload]
    return {"workload": workload, "encoding": enc, "shapes_out_in": shapes, "m": 1, "weights_per_shape": copies,
            "l2": "rotating distinct weights larger than 2x L2 per sweep", "activation": "fp32 N(0,1)",
            "weights": "N(0,0.02) packed on device, seeded"}


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from skainet_b200 import _lib as L, device

    rank, world, local = dist_env()
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    device.set_device(local)
    info = device.device_info()
    enc, shapes, bb, be = WORKLOADS[args.workload]
    per_sweep_one_copy = sum(algorithmic_bytes(bb, be, r, c) for r, c in shapes)
    copies = max(2, int(np.ceil(2.2 * info["l2_bytes"] / min(r * (c // be) * bb for r, c in shapes))))
    weights = [[device.Weight.synth(enc, r, c, seed=1000 * rank + 10 * si + ci, std=0.02) for ci in range(copies)]
               for si, (r, c) in enumerate(shapes)]
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(5 + rank)
    xs = [torch.randn(c, device="cuda", generator=gen, dtype=torch.float32) for _, c in shapes]
    ys = [torch.empty(r, device="cuda", dtype=torch.float32) for r, _ in shapes]
    launches_per_step = 0

    def sweep():
        n = 0
        for ci in range(copies):
            for si in range(len(shapes)):
                device.matmul(weights[si][ci], xs[si].data_ptr(), 1, ys[si].data_ptr(), L.ACT_NATIVE, sp)
                n += 2          # activation quantizer + matvec
        return n

    with torch.cuda.stream(stream):
        launches_per_step = sweep()          # allocates scratch outside capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            sweep()
    bytes_per_step = per_sweep_one_copy * copies

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------------------------------
    for _ in range(max(3, args.warmup)):
        with torch.cuda.stream(stream):
            graph.replay()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    # keep the GPU busy long enough for the clock sampler to see it under load
    if rank == 0 and not args.skip_cpu:
        t_end = time.time() + 1.0
        with torch.cuda.stream(stream):
            while time.time() < t_end:
                graph.replay(); stream.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the C ABI with host activations/outputs ----------------------------------
    hx = [torch.randn(c, dtype=torch.float32).pin_memory() for _, c in shapes]
    hy = [torch.empty(r, dtype=torch.float32).pin_memory() for r, _ in shapes]
    lib = L.lib()

    def e2e_sweep():
        for ci in range(copies):
            for si in range(len(shapes)):
                L.check(lib.skainet_cuda_memcpy_h2d(xs[si].data_ptr(), hx[si].data_ptr(), hx[si].numel() * 4, sp))
                device.matmul(weights[si][ci], xs[si].data_ptr(), 1, ys[si].data_ptr(), L.ACT_NATIVE, sp)
                L.check(lib.skainet_cuda_memcpy_d2h(hy[si].data_ptr(), ys[si].data_ptr(), hy[si].numel() * 4, sp))  # syncs

    e2e_steps = 0 if args.skip_e2e else max(1, min(args.steps, 5))
    for _ in range(0 if args.skip_e2e else 2):
        e2e_sweep()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(e2e_steps):
        e2e_sweep()
    e3.record(stream)
    barrier()
    e2e_ms = e2.elapsed_time(e3)

    t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peak, peak_kind = load_peaks()
        value = bytes_per_step * world * args.steps / (ms * 1e-3) / 1e9
        nmat = copies * len(shapes)
        per_launch_us = ms * 1e3 / (args.steps * nmat)
        achieved = (bytes_per_step / nmat) / (per_launch_us * 1e-6) / 1e9
        cpu = cpu_matvec_rate(args.workload, 10.0) if (world == 1 and not args.skip_cpu) else None
        line = {
            "metric": f"{args.workload}_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int4 -> int32, f32 accumulate" if enc == "Q4_K" else "int8 x int8 (2-term) -> int32, f32 accumulate",
            "data": "synthetic", "config": workload_config(args.workload, copies),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "q4k_matvec_kernel<1>" if enc == "Q4_K" else "q8_0_matvec_kernel<1>",
                         "avg_launch_us": per_launch_us,
                         "note": "avg launch = timed region / matvec launches (activation quantizer and launch gaps included)"},
            "e2e": {"value": (bytes_per_step * world * e2e_steps / (e2e_ms * 1e-3) / 1e9) if e2e_steps else None, "unit": "GB/s",
                    "h2d_bytes_per_step": int(sum(4 * c for _, c in shapes) * copies),
                    "d2h_bytes_per_step": int(sum(4 * r for r, _ in shapes) * copies),
                    "note": "weights resident; each matvec copies its activation in and its output out"},
            "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="q4k_matvec", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
