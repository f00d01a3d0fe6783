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


def step_err(got, ref):
    ref = np.asarray(ref, np.float64).reshape(-1); got = np.asarray(got, np.float64).reshape(-1)
    return float(np.abs(got - ref).max() / np.sqrt(np.mean(ref * ref)))


@pytest.mark.parametrize("shape", ["gqa64", "mha128_q8tables", "all_q4k"])
def test_teacher_forced_logits_and_tokens_match_cpu_composer(gpu, oracle, shape):
    """Both sides are fed the CPU composer's greedy tokens, so every step compares logits computed from
    the same tokens. The path has two rounding cliffs (binary16 K/V, int8 activations): an fp32
    rounding-order difference regularly lands on the other side of one (a cached K element moves by one
    f16 ulp, a few int8 activation codes by one), which moves logits by ~1e-2 of their RMS and stays in
    the cache. The reference's own two CPU builds drift apart the same way (tests/test_oracle.py), so the
    rel-1e-3 bar is checked per operator on identical inputs (next test); here: the drift stays at the
    cliff level and a token may differ only where the CPU's own margin is inside the step's error."""
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
    prompt = np.random.default_rng(9).integers(0, cfg.vocab, size=11)
    n_new = 12
    logits = None
    for t in prompt:
        logits = cpu.step(int(t))
    tok_gpu = m.prefill(prompt)
    errs = [step_err(m.logits(1)[0], logits)]
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)
    for _ in range(n_new):
        tok_cpu = oracle.argmax(logits)
        if tok_gpu != tok_cpu:
            gap = float(logits[tok_cpu] - logits[tok_gpu]) / float(np.sqrt(np.mean(logits ** 2)))
            assert gap <= 2 * errs[-1], f"token {tok_gpu} vs {tok_cpu}: CPU margin {gap:.2e} outside the step error {errs[-1]:.2e}"
        logits = cpu.step(tok_cpu)
        tin[0] = tok_cpu
        m.decode(tin, tout)
        tok_gpu = int(tout[0])
        errs.append(step_err(m.logits(1)[0], logits))
    assert max(errs) < 0.15, errs
    m.free()


def test_operators_inside_the_step_match_the_reference_on_the_same_inputs(gpu, oracle):
    """In-situ operator parity on a one-layer model: every stage the runtime leaves in its buffers is
    recomputed with the reference operator from the runtime's own upstream values. Bar: rel 1e-3 per
    stage. A stage whose input passes through RMSNorm/SwiGLU before the int8 activation quantizer can
    see a single code flip from a 1-ulp difference in that fp32 value (one flip moves the outputs by
    ~3e-3 of their RMS); such stages are counted, must stay rare, and must stay at the one-flip level."""
    from skainet_b200.llama import LlamaConfig
    R = oracle
    cfg = LlamaConfig(1, 512, 8, 4, 64, 1024, 1000, max_seq=64)
    m, W, _ = build(gpu, cfg, seed=21)
    use_ref = R.ref() is not None
    D, H, HK = 64, 8, 4
    ones = np.ones(512, np.float32)
    stages = []

    def stage(name, got, ref):
        stages.append((name, step_err(got, ref)))

    def mm(name, x, rows, cols):
        return R.matmul("Q4_K", x, W[(0, name)], cols, rows, "rm", use_ref=use_ref)
    Ks, Vs = [], []
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)
    for pos, t in enumerate([421, 870, 961, 286, 114, 7, 650, 33, 999, 12, 500, 77]):
        tin[0] = t
        m.decode(tin, tout)
        g_qkv, g_attn, g_gu, g_x = m.peek(1, 1024), m.peek(2, 512), m.peek(3, 2048), m.peek(0, 512)
        g_q = g_qkv[:512]
        x = R.dequant("Q8_0", W[(-1, "embed")][t * 34 * 16:(t + 1) * 34 * 16])
        xn = R.rms_norm(x, ones, 1e-5, use_ref=use_ref)
        # q in the buffer: as projected when the step rotates it inside its attention kernel, rotated in place otherwise
        q_ref = mm("q", xn, 512, 512)
        q_ref_rot = R.rope(q_ref.reshape(H, D), H, D, pos).reshape(-1)
        in_place = step_err(g_q, q_ref_rot) < step_err(g_q, q_ref)
        stage(f"q@{pos}", g_q, q_ref_rot if in_place else q_ref)
        q_rot = g_q.reshape(H, D) if in_place else R.rope(g_q.reshape(H, D), H, D, pos)
        stage(f"k@{pos}", g_qkv[512:768], mm("k", xn, 256, 512)); stage(f"v@{pos}", g_qkv[768:], mm("v", xn, 256, 512))
        # cache contents = binary16 of the runtime's own k (rotated) and v
        Ks.append(R.round_f16(R.rope(g_qkv[512:768].reshape(HK, D), HK, D, pos))); Vs.append(R.round_f16(g_qkv[768:].reshape(HK, D)))
        a = R.sdpa(q_rot.reshape(1, H, 1, D), np.stack(Ks, 1)[None], np.stack(Vs, 1)[None], 0.125, causal=True, use_ref=use_ref).reshape(-1)
        stage(f"attn@{pos}", g_attn, a)
        x1 = x + mm("o", g_attn, 512, 512)
        xn2 = R.rms_norm(x1, ones, 1e-5, use_ref=use_ref)
        stage(f"gate@{pos}", g_gu[:1024], mm("gate", xn2, 1024, 512)); stage(f"up@{pos}", g_gu[1024:], mm("up", xn2, 1024, 512))
        stage(f"x@{pos}", g_x, x1 + mm("down", R.swiglu(g_gu[:1024], g_gu[1024:]), 512, 1024))
        head = R.matmul("Q8_0", R.rms_norm(g_x, ones, 1e-5, use_ref=use_ref), W[(-1, "head")], 512, 1000, "rm", use_ref=use_ref)
        stage(f"logits@{pos}", m.logits(1)[0], head)
        assert int(tout[0]) == R.argmax(m.logits(1)[0])
    over = [(n, e) for n, e in stages if e > 1e-3]
    assert all(e < 2e-2 for _, e in over), over
    assert len(over) <= len(stages) // 10, over
    assert np.median([e for _, e in stages]) < 1e-4
    m.free()


def test_free_running_greedy_matches_until_a_near_tie(gpu, oracle):
    """Device-side greedy generation (graph replay, no host round trip) against the CPU composer's own
    greedy run: identical tokens, or a first divergence where the CPU's margin is inside the error."""
    from skainet_b200.llama import LlamaConfig
    from oracle.llama_cpu import CpuLlama
    cfg = LlamaConfig(2, 512, 8, 2, 64, 1024, 1000, max_seq=64)
    m, weights, gam = build(gpu, cfg, seed=5)
    cpu = CpuLlama(cfg, weights, gam)
    prompt = [3, 999, 17, 256, 4]
    want, want_logits = cpu.greedy(prompt, 10)
    first = m.prefill(prompt)
    got = [first] + [int(t) for t in m.generate([first], 9)[:, 0]]
    if got != want:
        i = next(k for k in range(10) if got[k] != want[k])
        lg = want_logits[i]
        gap = float(lg[want[i]] - lg[got[i]]) / float(np.sqrt(np.mean(lg ** 2)))
        assert gap < 0.05, f"diverged at step {i}: GPU {got[i]} vs CPU {want[i]} with CPU margin {gap:.3f} of logit RMS"
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


def test_decode_reports_a_bounded_wait_that_ran_out(gpu, cuda_lib):
    """No fault involved: the self-test kernel waits on a barrier nothing completes, gives up and raises the device
    flag. The next synchronising runtime call must report SKAINET_CUDA_ERR_TIMEOUT instead of returning tokens as if
    nothing had happened, clear the condition, and work again afterwards."""
    import ctypes as C
    from skainet_b200.llama import Llama, LlamaConfig
    from skainet_b200._lib import SkainetCudaError, ERR_TIMEOUT
    m = Llama(LlamaConfig(1, 256, 4, 2, 64, 512, 300, max_seq=32))
    m.synth(); m.finalize()
    tin, tout = np.array([5], np.int32), np.zeros(1, np.int32)
    m.decode(tin, tout)
    good = int(tout[0])
    outcome = C.c_int32(0)
    assert cuda_lib.skainet_cuda_selftest_bounded_wait(C.byref(outcome)) == 0 and outcome.value == 2
    with pytest.raises(SkainetCudaError) as e:
        m.decode(tin, tout)
    assert e.value.status == ERR_TIMEOUT and "bounded wait" in str(e.value)
    assert cuda_lib.skainet_cuda_device_status() == 0          # the call cleared the condition
    m.reset()
    m.decode(tin, tout)
    assert int(tout[0]) == good
    m.free()


def test_prefill_and_decode_are_bit_repeatable(gpu):
    """Three runs of the same request (a 300-token prompt through the tcgen05 / mma.sync tile kernels and the
    tensor-core prefill attention, then 48 greedy tokens through the ring matvecs and split-K attention) give identical
    logits bit for bit and identical tokens: every reduction in the path has a fixed order, and a race between the
    warp roles of a kernel would show up as a run that differs."""
    from skainet_b200.llama import Llama, LlamaConfig
    from skainet_b200 import _lib
    cfg = LlamaConfig(3, 2048, 16, 4, 128, 5632, 4000, max_seq=512)
    m = Llama(cfg)
    m.synth(seed=21, std=0.03)
    m.finalize()
    prompt = list(np.random.default_rng(8).integers(0, cfg.vocab, size=300))
    runs = []
    for _ in range(3):
        m.reset()
        f = m.prefill(prompt)
        lg = m.logits(1).copy()
        toks = [f] + list(m.generate([f], 48)[:, 0])
        runs.append((lg, toks, m.logits(1).copy()))
    for lg, toks, lg2 in runs[1:]:
        np.testing.assert_array_equal(lg, runs[0][0])
        assert toks == runs[0][1]
        np.testing.assert_array_equal(lg2, runs[0][2])
    assert np.isfinite(runs[0][0]).all()
    assert _lib.lib().skainet_cuda_device_status() == 0
    m.free()
