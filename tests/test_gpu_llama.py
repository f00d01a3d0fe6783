"""GPU parity of the decoder runtime against the CPU composer built from the reference's operators:
identical greedy tokens and logits within rel 1e-3, on a scaled-down Llama-style model."""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu

NAMES = {"q": 4, "k": 5, "v": 6, "o": 7, "gate": 9, "up": 10, "down": 11}


def build(gpu, cfg, seed=100, norms=False):
    from skainet_b200.llama import Llama, W_EMBED, W_HEAD, W_ATTN_NORM, W_FFN_NORM, W_OUT_NORM
    m = Llama(cfg)
    m.synth(seed=seed, std=0.05)
    gam = {}
    if norms:
        rng = np.random.default_rng(seed)
        for l in range(cfg.n_layers):
            for name, which in (("attn_norm", W_ATTN_NORM), ("ffn_norm", W_FFN_NORM)):
                gam[(l, name)] = (1 + 0.2 * rng.standard_normal(cfg.d_model)).astype(np.float32)
                m.set_norm(l, which, gam[(l, name)])
        gam[(-1, "out_norm")] = (1 + 0.2 * rng.standard_normal(cfg.d_model)).astype(np.float32)
        m.set_norm(0, W_OUT_NORM, gam[(-1, "out_norm")])
    weights = {(-1, "embed"): m.export_weight(0, W_EMBED), (-1, "head"): m.export_weight(0, W_HEAD)}
    for l in range(cfg.n_layers):
        for name, which in NAMES.items():
            weights[(l, name)] = m.export_weight(l, which)
    m.finalize()
    return m, weights, gam


@pytest.mark.parametrize("shape", ["gqa64", "mha128_q8tables", "all_q4k"])
def test_greedy_tokens_and_logits_match_cpu_composer(gpu, oracle, shape):
    from skainet_b200.llama import LlamaConfig
    from oracle.llama_cpu import CpuLlama
    if shape == "gqa64":
        cfg = LlamaConfig(2, 512, 8, 4, 64, 1024, 1000, max_seq=64)
    elif shape == "mha128_q8tables":
        cfg = LlamaConfig(2, 512, 4, 4, 128, 768, 777, max_seq=64, rope_mode=1)
    else:
        cfg = LlamaConfig(1, 256, 4, 1, 64, 512, 515, max_seq=300, table_enc="Q4_K")
    m, weights, gam = build(gpu, cfg, norms=True)
    cpu = CpuLlama(cfg, weights, gam)
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, cfg.vocab, size=11)
    n_new = 12
    want_tokens, want_logits = cpu.greedy(prompt, n_new)

    first = m.prefill(prompt)
    assert first == want_tokens[0]
    got = m.generate([first], n_new - 1)[:, 0]
    assert [first] + list(got) == want_tokens, f"GPU {[first] + list(got)} vs CPU {want_tokens}"
    # logits of the last device step are those the CPU composer computes after feeding the last generated token
    rel_err_ok(m.logits(1)[0], cpu.step(want_tokens[-1]))
    m.free()


def test_logits_after_prefill_and_each_step(gpu, oracle):
    from skainet_b200.llama import LlamaConfig
    from oracle.llama_cpu import CpuLlama
    cfg = LlamaConfig(2, 512, 8, 2, 64, 1024, 1000, max_seq=64)
    m, weights, gam = build(gpu, cfg, seed=5)
    cpu = CpuLlama(cfg, weights, gam)
    prompt = [3, 999, 17, 256, 4]
    logits = None
    for t in prompt:
        logits = cpu.step(t)
    tok = m.prefill(prompt)
    assert tok == oracle.argmax(logits)
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)
    for _ in range(6):
        tin[0] = tok
        m.decode(tin, tout)                       # host token in, host token out
        logits = cpu.step(tok)
        rel_err_ok(m.logits(1)[0], logits)        # rel 1e-3, scale-aware
        assert int(tout[0]) == oracle.argmax(logits)
        tok = int(tout[0])
    m.free()


def test_batched_sequences_equal_single_runs_and_reset(gpu):
    from skainet_b200.llama import LlamaConfig
    cfg = LlamaConfig(2, 512, 8, 4, 64, 1024, 1000, max_seq=64, max_batch=3)
    m, _, _ = build(gpu, cfg, seed=11)
    prompts = [[1, 2, 3, 4, 5, 6], [9, 8, 7], [100, 200, 300, 400]]
    singles = []
    for p in prompts:
        m.reset()
        f = m.prefill(p, seq=0)
        singles.append([f] + list(m.generate([f], 5)[:, 0]))
    m.reset()
    firsts = [m.prefill(p, seq=i) for i, p in enumerate(prompts)]
    out = m.generate(firsts, 5)
    for i in range(3):
        assert [firsts[i]] + list(out[:, i]) == singles[i]
    m.free()


def test_context_bucket_boundary_and_prefill_chunks(gpu):
    """A prompt longer than one prefill chunk and a decode that crosses the 256-key bucket boundary give
    the same tokens as feeding the tokens one by one."""
    from skainet_b200.llama import LlamaConfig
    cfg = LlamaConfig(1, 256, 4, 2, 64, 512, 300, max_seq=600)
    m, _, _ = build(gpu, cfg, seed=3)
    rng = np.random.default_rng(1)
    prompt = list(rng.integers(0, 300, size=270))
    f = m.prefill(prompt)
    a = [f] + list(m.generate([f], 8)[:, 0])
    m.reset()
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)
    for t in prompt:
        tin[0] = t
        m.decode(tin, tout)
    b = [int(tout[0])] + list(m.generate([int(tout[0])], 8)[:, 0])
    assert a == b
    m.free()


def test_runtime_argument_errors(gpu):
    from skainet_b200.llama import Llama, LlamaConfig
    with pytest.raises(ValueError):
        Llama(LlamaConfig(1, 256, 4, 3, 64, 512, 300))            # heads not a multiple of kv heads
    m = Llama(LlamaConfig(1, 256, 4, 2, 64, 512, 300, max_seq=16))
    with pytest.raises(ValueError, match="finalize"):
        m.prefill([1, 2, 3])
    m.synth(); m.finalize()
    with pytest.raises(ValueError, match="max_seq"):
        m.prefill(list(range(17)))
    m.free()
