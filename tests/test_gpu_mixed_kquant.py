"""A K-quant model that mixes Q6_K tensors in among its Q4_K ones, the way real Q4_K_M files do (attn_v, ffn_down and
the output head as Q6_K): the runtime takes the Q6_K tensors through skainet_cuda_llama_set_weight, runs q|k merged and
v separately where their encodings differ, and its logits follow the CPU composer that calls the reference's
q4k / q6k kernels (native/src/q4k_matmul.c, native/src/q6k_matmul.c) on the same bytes."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NAMES = {"q": 4, "k": 5, "v": 6, "o": 7, "gate": 9, "up": 10, "down": 11}


def q6k_blocks(oracle, rows, cols, seed, d_scale=6e-5):
    blk = oracle.random_kquant_blocks("Q6_K", rows, cols, seed=seed).reshape(-1, 210)
    rng = np.random.default_rng(seed + 1)
    blk[:, 208:210] = np.abs(d_scale * (1 + 0.3 * rng.standard_normal(blk.shape[0]))).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return blk.reshape(-1)


@pytest.mark.parametrize("mixed_v", [True, False])
def test_mixed_q4k_q6k_model_follows_the_cpu_composer(gpu, oracle, mixed_v):
    from skainet_b200.llama import Llama, LlamaConfig, W_EMBED, W_HEAD, W_V, W_DOWN
    from oracle.llama_cpu import CpuLlama
    cfg = LlamaConfig(2, 512, 8, 4, 64, 1024, 1000, max_seq=64, table_enc="Q4_K")
    m = Llama(cfg)
    m.synth(seed=31, std=0.05)
    weights, encs = {}, {}
    # Q6_K in place of ffn_down of layer 1, the output head, and (first variant) attn_v of every layer
    repl = [(1, "down", W_DOWN, 512, 1024), (-1, "head", W_HEAD, 1000, 512)]
    if mixed_v:
        repl += [(l, "v", W_V, 256, 512) for l in range(2)]
    for layer, name, which, rows, cols in repl:
        packed = q6k_blocks(oracle, rows, cols, seed=100 + 7 * layer + which)
        m.set_weight(max(layer, 0), which, gpu.Weight.upload(packed, "Q6_K", rows, cols))
        weights[(layer, name)], encs[(layer, name)] = packed, "Q6_K"
    weights.setdefault((-1, "embed"), m.export_weight(0, W_EMBED))
    for l in range(2):
        for name, which in NAMES.items():
            weights.setdefault((l, name), m.export_weight(l, which))
    m.finalize()
    cpu = CpuLlama(cfg, weights, {}, encs=encs)
    prompt = [5, 900, 17, 333, 64, 2, 811]
    logits = None
    for t in prompt:
        logits = cpu.step(t)
    m.prefill(prompt)
    errs = []
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)
    for _ in range(8):
        got = m.logits(1)[0].astype(np.float64)
        ref = logits.astype(np.float64)
        errs.append(float(np.abs(got - ref).max() / np.sqrt(np.mean(ref * ref))))
        tok = oracle.argmax(logits)
        logits = cpu.step(tok)
        tin[0] = tok
        m.decode(tin, tout)
    # the same bar as the teacher-forced test of the single-encoding models: drift stays at the level of single rounding flips
    assert max(errs) < 0.15 and np.median(errs) < 0.02, errs
    # batched rows (prefill chunk) and single rows agree: the part-wise projections scatter into the merged layout correctly
    m.reset()
    for t in prompt:
        tin[0] = t
        m.decode(tin, tout)
    a = m.logits(1)[0].copy()
    m.reset()
    m.prefill(prompt)
    b = m.logits(1)[0]
    assert float(np.abs(a - b).max() / np.sqrt(np.mean(a.astype(np.float64) ** 2))) < 0.05
    from skainet_b200 import _lib
    assert _lib.lib().skainet_cuda_device_status() == 0
    m.free()
