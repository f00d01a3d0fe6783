"""The device KV-cache store against the restatement of the reference's DefaultKvCacheStore, on the scenarios the
reference's own ring tests use (skainet-lang/skainet-lang-core/src/commonTest/kotlin/sk/ainet/lang/memory/
WindowedKvTest.kt:29-150: per-token contents that identify their position, a cache of four slots filled with six,
seven and ten tokens). CPU tests pin the restatement on those scenarios; GPU tests compare the store with it."""
import numpy as np
import pytest

from conftest import rel_err_ok

HEADS = 2


def token(step, head_dim, offset=0.0):
    # every element identifies its position: (step * 100 + i) * 0.01 + offset  (WindowedKvTest.kt:32-33)
    return ((step * 100 + np.arange(HEADS * head_dim)) * 0.01 + offset).astype(np.float32)


def fill(store, steps, head_dim, first=0):
    for step in range(first, first + steps):
        store.appendToken(0, token(step, head_dim), token(step, head_dim, 0.5))


# ---- the restatement on the reference's scenarios (CPU) ----------------------------------------------------------
def test_restatement_non_sliding_cache_refuses_to_overflow():
    from oracle.kv_store import CpuKvStore
    s = CpuKvStore(1, HEADS, 4, 4)
    fill(s, 4, 4)
    with pytest.raises(RuntimeError, match="KV cache is full"):
        s.appendToken(0, token(4, 4), token(4, 4))
    assert s.windowStart == 0


def test_restatement_ring_keeps_the_newest_and_reads_in_position_order():
    from oracle.kv_store import CpuKvStore
    s = CpuKvStore(1, HEADS, 4, 4, slidingWindow=True)
    fill(s, 6, 4)
    assert s.currentSeqLen == 6 and s.windowStart == 2
    with pytest.raises(ValueError):
        s.readKeys(0, 0, 6)
    fill(s, 1, 4, first=6)
    flat = s.readKeys(0, 3, 7)
    for index, step in enumerate([3, 4, 5, 6]):
        np.testing.assert_array_equal(flat[:, index, :].reshape(-1), token(step, 4))


def test_restatement_wrapped_attention_equals_the_flat_run():
    from oracle.kv_store import CpuKvStore, windowed_decode_step
    ring = CpuKvStore(1, HEADS, 4, 4, slidingWindow=True)
    fill(ring, 10, 4)
    flat = CpuKvStore(1, HEADS, 4, 64)
    fill(flat, 4, 4, first=6)
    q = (0.1 * (np.arange(HEADS * 4) + 1)).astype(np.float32)
    a = windowed_decode_step(q, ring.readKeys(0, 6, 10), ring.readValues(0, 6, 10))
    b = windowed_decode_step(q, flat.readKeys(0, 0, 4), flat.readValues(0, 0, 4))
    np.testing.assert_array_equal(a, b)
    # and the online softmax is the softmax
    k, v = flat.readKeys(0, 0, 4).astype(np.float64), flat.readValues(0, 0, 4).astype(np.float64)
    sc = np.einsum("hd,hpd->hp", q.reshape(HEADS, 4).astype(np.float64), k) / 2.0
    p = np.exp(sc - sc.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    np.testing.assert_allclose(a, np.einsum("hp,hpd->hd", p, v), rtol=1e-5)


def test_restatement_evict_truncates_and_zeroes():
    from oracle.kv_store import CpuKvStore
    s = CpuKvStore(2, HEADS, 4, 8)
    for step in range(5):
        for layer in range(2):
            s.appendToken(layer, token(step, 4), token(step, 4, 0.5))
    assert s.currentSeqLen == 5
    s.evict(3)
    assert s.currentSeqLen == 3 and not s.keys[:, :, 3:, :].any()
    with pytest.raises(ValueError):
        s.evict(4)


# ---- the device store against the restatement (GPU) ------------------------------------------------------------------
def _pair(gpu, layers, head_dim, max_seq, sliding):
    from oracle.kv_store import CpuKvStore
    from skainet_b200.kvstore import DeviceKvCacheStore
    return DeviceKvCacheStore(layers, HEADS, head_dim, max_seq, sliding), CpuKvStore(layers, HEADS, head_dim, max_seq, sliding, f16=True)


@pytest.mark.gpu
def test_device_store_append_read_ring_and_refusals(gpu):
    D = 64
    dev, cpu = _pair(gpu, 1, D, 4, True)
    for s in (dev, cpu):
        fill(s, 6, D)
    assert dev.currentSeqLen == cpu.currentSeqLen == 6 and dev.windowStart == cpu.windowStart == 2
    with pytest.raises(ValueError):
        dev.readKeys(0, 0, 6)                               # position 0 was overwritten
    with pytest.raises(ValueError):
        dev.readKeys(0, 3, 7)                               # beyond the sequence
    for s in (dev, cpu):
        fill(s, 1, D, first=6)
    np.testing.assert_array_equal(dev.readKeys(0, 3, 7), cpu.readKeys(0, 3, 7))      # across the wrap, oldest first
    np.testing.assert_array_equal(dev.readValues(0, 3, 7), cpu.readValues(0, 3, 7))
    np.testing.assert_array_equal(dev.readKeys(0, 4), cpu.readKeys(0, 4))
    assert dev.physicalBytes == 2 * 1 * HEADS * 4 * D * 2
    dev.free()
    full, _ = _pair(gpu, 1, D, 4, False)
    fill(full, 4, D)
    with pytest.raises(ValueError, match="KV cache is full"):
        full.appendToken(0, token(4, D), token(4, D))
    with pytest.raises(ValueError, match="Key size mismatch"):
        full.appendToken(0, np.zeros(3, np.float32), token(4, D))
    full.free()


@pytest.mark.gpu
def test_device_store_layers_advance_with_the_last_layer_evict_and_clear(gpu):
    D = 64
    dev, cpu = _pair(gpu, 3, D, 8, False)
    rng = np.random.default_rng(3)
    for step in range(5):
        for layer in range(3):
            k, v = rng.standard_normal(HEADS * D).astype(np.float32), rng.standard_normal(HEADS * D).astype(np.float32)
            dev.appendToken(layer, k, v); cpu.appendToken(layer, k, v)
            assert dev.currentSeqLen == cpu.currentSeqLen
    for layer in range(3):
        np.testing.assert_array_equal(dev.readKeys(layer), cpu.readKeys(layer))
        np.testing.assert_array_equal(dev.readValues(layer, 1, 4), cpu.readValues(layer, 1, 4))
    dev.evict(3); cpu.evict(3)
    assert dev.currentSeqLen == 3
    with pytest.raises(ValueError):
        dev.evict(4)
    k, v = np.ones(HEADS * D, np.float32), np.full(HEADS * D, 2.0, np.float32)
    for layer in range(3):
        dev.appendToken(layer, k, v); cpu.appendToken(layer, k, v)
    np.testing.assert_array_equal(dev.readKeys(1), cpu.readKeys(1))
    dev.clear()
    assert dev.currentSeqLen == 0
    dev.free()


@pytest.mark.gpu
@pytest.mark.parametrize("D,qheads,cap,steps,window", [(64, 2, 4, 10, 4), (128, 8, 48, 130, 48), (128, 4, 300, 777, 200), (64, 16, 512, 400, 400)])
def test_attention_over_a_wrapped_window_reads_the_ring_in_place(gpu, oracle, D, qheads, cap, steps, window):
    """The ring has wrapped (or not: last case); attention over its newest `window` positions must equal the reference
    SDPA over the same positions read out in order, and a cache that never wrapped must give the same bits."""
    dev, cpu = _pair(gpu, 1, D, cap, True)
    flat, _ = _pair(gpu, 1, D, max(steps, cap), False)
    rng = np.random.default_rng(D + steps)
    for step in range(steps):
        k, v = rng.standard_normal(HEADS * D).astype(np.float32), rng.standard_normal(HEADS * D).astype(np.float32)
        dev.appendToken(0, k, v); cpu.appendToken(0, k, v); flat.appendToken(0, k, v)
    frm, to = steps - window, steps
    assert frm >= dev.windowStart
    q = rng.standard_normal((qheads, D)).astype(np.float32)
    dq, dout, dout2 = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer(q.nbytes), gpu.DeviceBuffer(q.nbytes)
    dev.decodeStep(0, dq.ptr, dout.ptr, qheads, frm, to)
    flat.decodeStep(0, dq.ptr, dout2.ptr, qheads, frm, to)
    got, got_flat = dout.download(np.float32, q.size).reshape(qheads, D), dout2.download(np.float32, q.size).reshape(qheads, D)
    K, V = cpu.readKeys(0, frm, to), cpu.readValues(0, frm, to)
    ref = oracle.sdpa(q.reshape(1, qheads, 1, D), K[None], V[None], float(1.0 / np.sqrt(D)), causal=True,
                      use_ref=oracle.ref() is not None)[0, :, 0, :]
    rel_err_ok(got, ref)
    rel_err_ok(got_flat, ref)
    if window <= 16:      # the reference's own loop (online softmax, oldest first) on the small case
        from oracle.kv_store import windowed_decode_step
        g = qheads // HEADS
        rel_err_ok(got, windowed_decode_step(q, np.repeat(K, g, axis=0), np.repeat(V, g, axis=0)))
    with pytest.raises(ValueError):
        dev.decodeStep(0, dq.ptr, dout.ptr, qheads, max(0, dev.windowStart - 1) if dev.windowStart > 0 else -1, to)
    dev.free(); flat.free()


@pytest.mark.gpu
def test_token_in_flight_counts_before_the_last_layer_is_appended(gpu, oracle):
    D = 64
    dev, cpu = _pair(gpu, 2, D, 16, False)
    rng = np.random.default_rng(8)
    def tok():
        return rng.standard_normal(HEADS * D).astype(np.float32), rng.standard_normal(HEADS * D).astype(np.float32)
    for step in range(5):
        for layer in range(2):
            k, v = tok(); dev.appendToken(layer, k, v); cpu.appendToken(layer, k, v)
    k, v = tok()
    dev.appendToken(0, k, v); cpu.appendToken(0, k, v)          # layer 0 of token 5; the length is still 5
    assert dev.currentSeqLen == 5
    q = rng.standard_normal((HEADS, D)).astype(np.float32)
    dq, dout = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer(q.nbytes)
    dev.decodeStep(0, dq.ptr, dout.ptr, HEADS, 0, 6)
    K, V = cpu.keys[0][:, :6, :], cpu.values[0][:, :6, :]
    ref = oracle.sdpa(q.reshape(1, HEADS, 1, D), K[None], V[None], 0.125, causal=True)[0, :, 0, :]
    rel_err_ok(dout.download(np.float32, q.size).reshape(HEADS, D), ref)
    with pytest.raises(ValueError):
        dev.decodeStep(0, dq.ptr, dout.ptr, HEADS, 0, 7)
    dev.free()
