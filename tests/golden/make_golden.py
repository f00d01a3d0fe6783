"""Generates the committed fixtures under tests/golden/ from the reference itself.

Run where the reference tree is mounted (it is not present on the GPU box):

    python tests/golden/make_golden.py [/path/to/reference]

Writes
  reference_digests.json — the digest strings the reference's golden tests record for this path
      (skainet-backends/skainet-backend-cpu/src/goldenTest/kotlin/sk/ainet/exec/golden/Goldens.kt),
      read from the source file as text;
  ref_vectors.npz — seeded inputs and the outputs of the reference's own compiled C kernels
      (oracle/_ref, built by oracle/Makefile) for the matvec, RMSNorm, SDPA and SiLU entry points.
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import ref as R  # noqa: E402

KEYS = ["decode/Q4_K", "decode/Q8_0", "decode/Q5_K", "decode/Q6_K", "scalar-matmul/Q4_K", "scalar-matmul/Q8_0",
        "dispatch-bridge/Q4_K", "dispatch-bridge/Q8_0"] + [f"turboquant/{t}/{k}" for t in ("polar4", "polar3", "polar4-qjl1") for k in ("codes", "scales", "decoded")]


def digests(ref_root: str) -> dict:
    path = os.path.join(ref_root, "skainet-backends/skainet-backend-cpu/src/goldenTest/kotlin/sk/ainet/exec/golden/Goldens.kt")
    text = open(path).read()
    out = {}
    for k in KEYS:
        m = re.search(r'"%s" to "([^"]+)"' % re.escape(k), text)
        assert m, k
        out[k] = m.group(1)
    return out


def vectors() -> dict:
    assert R.ref() is not None, "oracle/_ref is not built"
    rng = np.random.Generator(np.random.PCG64(20240601))
    v = {}
    # Q4_K / Q8_0 matvec, row-major and feed order, incl. a non-multiple-of-8 row count and K = 43 blocks-like tail
    for enc, k, n in (("Q4_K", 1024, 37), ("Q4_K", 2816, 16), ("Q8_0", 512, 45), ("Q8_0", 96, 7)):
        w = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
        packed = R.quantize_q4k(w) if enc == "Q4_K" else R.quantize_q8_0(w)
        x = rng.standard_normal(k).astype(np.float32)
        y_rm = R.matmul(enc, x, packed, k, n, "rm", use_ref=True)
        y_feed = R.matmul(enc, x, R.to_feed_order(packed, enc, n, k), k, n, "feed", use_ref=True)
        tag = f"{enc}_{k}x{n}"
        v[tag + "_w"] = packed; v[tag + "_x"] = x; v[tag + "_y_rm"] = y_rm; v[tag + "_y_feed"] = y_feed
    # RMSNorm
    x = rng.standard_normal((3, 320)).astype(np.float32); g = rng.standard_normal(320).astype(np.float32)
    v["rms_x"] = x; v["rms_g"] = g; v["rms_y"] = R.rms_norm(x, g, 1e-5, use_ref=True)
    # SDPA: GQA decode (seq_q = 1) and a short causal prefill with a sliding window
    q = rng.standard_normal((2, 8, 1, 64)).astype(np.float32)
    k = rng.standard_normal((2, 2, 40, 64)).astype(np.float32); vv = rng.standard_normal((2, 2, 40, 64)).astype(np.float32)
    v["sdpa_dec_q"] = q; v["sdpa_dec_k"] = k; v["sdpa_dec_v"] = vv
    v["sdpa_dec_o"] = R.sdpa(q, k, vv, 0.125, causal=True, use_ref=True)
    q = rng.standard_normal((1, 4, 9, 32)).astype(np.float32)
    k = rng.standard_normal((1, 2, 9, 32)).astype(np.float32); vv = rng.standard_normal((1, 2, 9, 32)).astype(np.float32)
    v["sdpa_win_q"] = q; v["sdpa_win_k"] = k; v["sdpa_win_v"] = vv
    v["sdpa_win_o"] = R.sdpa(q, k, vv, 0.2, causal=True, window=4, use_ref=True)
    # SiLU
    x = (4 * rng.standard_normal(257)).astype(np.float32)
    v["silu_x"] = x; v["silu_y"] = R.silu(x, use_ref=True)
    return v


if __name__ == "__main__":
    # the reference checkout: argument, else SKAINET_REFERENCE_ROOT, else a directory `reference` beside this repository
    ref_root = (sys.argv[1] if len(sys.argv) > 1 else
                os.environ.get("SKAINET_REFERENCE_ROOT", os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference"))))
    json.dump(digests(ref_root), open(os.path.join(HERE, "reference_digests.json"), "w"), indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **vectors())
    print("wrote", os.listdir(HERE))
