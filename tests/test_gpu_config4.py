"""Greedy-token parity at full width: the 7B-class shape of benchmark config 4 (d 4096, FFN 11008, 32 heads of 128,
vocab 32000, Q4_K linears, Q8_0 embedding / output, N(0, 0.02) seeded) against the CPU composer built from the
reference's own C kernels on the exported bytes.

What is asserted: the free-running greedy tokens are identical up to the first step at which the CPU's own margin
between the two candidate tokens is inside that step's measured GPU-vs-CPU logit error (a near tie that any second
implementation of this arithmetic may resolve the other way), or for the whole run if no such step occurs; and the
teacher-forced logit error (both sides fed the CPU's tokens) stays inside the distance between the reference's own two
CPU builds on the same tokens (the control: SKAINET_PARITY_CONTROL steps of the strict-fp32 restatement, 4 by default). The default run uses 4 of the 32 layers (every kernel at its full-width shape: ring matvecs for the 25 MB
FFN weights and the 139 MB Q8_0 head, one-tile kernels for the 9 MB attention weights, tile kernels for the prompt).
SKAINET_FULL_CONFIG4=1 runs all 32 layers with the 64-token prompt + 128 tokens; SKAINET_PARITY_REPORT=<file> writes
the per-step numbers as JSON.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NAMES = {"q": 4, "k": 5, "v": 6, "o": 7, "gate": 9, "up": 10, "down": 11}


def run_token_parity(gpu, oracle, n_layers: int, n_prompt: int, n_new: int, n_control: int = 0) -> dict:
    from skainet_b200.llama import Llama, LlamaConfig, W_EMBED, W_HEAD
    from oracle.llama_cpu import CpuLlama
    cfg = LlamaConfig.llama7b(max_seq=n_prompt + n_new + 8)
    cfg.n_layers = n_layers
    m = Llama(cfg)
    m.synth(seed=100, std=0.02)
    weights = {(-1, "embed"): m.export_weight(0, W_EMBED), (-1, "head"): m.export_weight(0, W_HEAD)}
    for l in range(n_layers):
        for name, which in NAMES.items():
            weights[(l, name)] = m.export_weight(l, which)
    m.finalize()
    cpu = CpuLlama(cfg, weights, {})
    prompt = np.random.default_rng(9).integers(0, cfg.vocab, size=n_prompt)
    cpu_tokens, cpu_logits = cpu.greedy(prompt, n_new)
    # control: the reference's OTHER CPU build of the same algorithm (the strict-fp32 restatement instead of the
    # -ffast-math C) fed the same tokens: how far two CPU implementations drift apart on this model
    control, control_div = [], None
    if n_control > 0 and oracle.ref() is not None:
        other = CpuLlama(cfg, weights, {}, use_ref=False)
        lg = None
        for t in prompt:
            lg = other.step(int(t))
        for i in range(min(n_control, n_new)):
            ref = cpu_logits[i].astype(np.float64)
            control.append(float(np.abs(lg.astype(np.float64) - ref).max() / np.sqrt(np.mean(ref * ref))))
            if control_div is None and oracle.argmax(lg) != cpu_tokens[i]:
                control_div = i               # the other CPU build would have picked another token here
            if i + 1 < min(n_control, n_new):
                lg = other.step(int(cpu_tokens[i]))
    # free-running on the device
    first = m.prefill(prompt)
    gpu_tokens = [first] + [int(t) for t in m.generate([first], n_new - 1)[:, 0]]
    # teacher-forced: the CPU's tokens on both sides
    m.reset()
    m.prefill(prompt)
    errs, margins = [], []
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)
    for i in range(n_new):
        lg = m.logits(1)[0].astype(np.float64)
        ref = cpu_logits[i].astype(np.float64)
        rms = float(np.sqrt(np.mean(ref * ref)))
        errs.append(float(np.abs(lg - ref).max() / rms))
        srt = np.sort(ref)
        margins.append(float((srt[-1] - srt[-2]) / rms))
        tin[0] = cpu_tokens[i]
        m.decode(tin, tout)
    div = next((i for i in range(n_new) if gpu_tokens[i] != cpu_tokens[i]), None)
    out = {"layers": n_layers, "prompt_tokens": n_prompt, "generated": n_new, "first_divergence": div,
           "teacher_forced_rel_logit_err": {"max": max(errs), "median": float(np.median(errs)), "per_step": errs},
           "cpu_builds_rel_logit_err": {"max": max(control) if control else None, "per_step": control, "first_token_difference": control_div},
           "cpu_top2_margin": {"min": min(margins), "per_step": margins}, "cpu_tokens": [int(t) for t in cpu_tokens], "gpu_tokens": gpu_tokens}
    if div is not None:
        ref = cpu_logits[div].astype(np.float64)
        rms = float(np.sqrt(np.mean(ref * ref)))
        out["divergence"] = {"step": div, "cpu_token": int(cpu_tokens[div]), "gpu_token": int(gpu_tokens[div]),
                             "cpu_margin_between_them": float((ref[cpu_tokens[div]] - ref[gpu_tokens[div]]) / rms),
                             "gpu_vs_cpu_logit_err_at_step": errs[div]}
    from skainet_b200 import _lib
    out["device_status"] = int(_lib.lib().skainet_cuda_device_status())
    m.free()
    return out


def check(report: dict) -> None:
    assert report["device_status"] == 0
    errs = report["teacher_forced_rel_logit_err"]
    assert np.isfinite(errs["per_step"]).all()
    ctl = report["cpu_builds_rel_logit_err"]["per_step"]
    if ctl:
        # The yardstick is the reference against itself: its -ffast-math C and its strict-fp32 restatement, fed the same
        # tokens, end up this far apart on this model (every int8 activation quantizer turns a relative input difference e
        # into about 0.15 * sqrt(e) at its output, so any two implementations settle a few percent apart). The GPU must
        # sit inside that envelope, on the steps the control covers and over the whole run.
        assert max(errs["per_step"][:len(ctl)]) <= 1.5 * max(ctl), (errs["per_step"][:len(ctl)], ctl)
        assert errs["max"] <= 2.0 * max(ctl), (errs["max"], max(ctl))
    else:
        assert errs["max"] < 0.5
    if report["first_divergence"] is not None:
        d = report["divergence"]
        assert d["cpu_margin_between_them"] <= 2.0 * d["gpu_vs_cpu_logit_err_at_step"], (
            f"tokens diverge at step {d['step']} with a CPU margin of {d['cpu_margin_between_them']:.3e} of the logit RMS, "
            f"outside the measured error {d['gpu_vs_cpu_logit_err_at_step']:.3e}")


def test_full_width_token_parity(gpu, oracle):
    full = os.environ.get("SKAINET_FULL_CONFIG4") == "1"
    report = run_token_parity(gpu, oracle, 32 if full else 4, 64 if full else 16, 128 if full else 32, n_control=int(os.environ.get("SKAINET_PARITY_CONTROL", "4")))
    path = os.environ.get("SKAINET_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(report, f)
    summary = {k: report[k] for k in ("layers", "first_divergence")}
    summary["err_max"] = report["teacher_forced_rel_logit_err"]["max"]
    summary["margin_min"] = report["cpu_top2_margin"]["min"]
    print("config-4 token parity:", json.dumps(summary), json.dumps(report.get("divergence")))
    check(report)
