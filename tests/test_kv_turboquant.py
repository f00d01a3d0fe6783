"""The TurboQuant codec and KV store on the GPU against the restatement pinned to the reference's golden digests
(oracle/turboquant.py, tests/test_turboquant_oracle.py). Bar: bit-exact — encoded bytes, scales, residuals and decoded
values are integer / single-rounding fp32 work in a fixed order; attention over the decoded window: rel 1e-3."""
import json
import os

import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
DIGESTS = json.load(open(os.path.join(HERE, "golden", "reference_digests.json")))


def byte_digest(R, b):
    b = np.asarray(b, np.uint8)
    return f"n={b.size} fnv={R.fnv1a64(b.tobytes()):016x} head=" + "".join(f"{int(x):02x}" for x in b[:8])


@pytest.mark.parametrize("tag,bits,qjl,rbits", [("polar4", 4, False, 1), ("polar3", 3, False, 1), ("polar4-qjl1", 4, True, 1)])
def test_codec_reproduces_the_reference_golden_digests(gpu, oracle, tag, bits, qjl, rbits):
    """TurboQuantGoldenTest.kt:15-22 through the C ABI: 128 seeded floats x 3, seed 7."""
    from skainet_b200.kvstore import TurboQuantCodec, TurboQuantConfig
    x = oracle.golden_floats(128, 0x5EED0003, 3.0)
    blk = TurboQuantCodec.encode(x, TurboQuantConfig(bits, qjl, rbits, 7))
    assert byte_digest(oracle, blk["packedCodes"]) == DIGESTS[f"turboquant/{tag}/codes"]
    assert oracle.golden_digest(blk["scales"]) == DIGESTS[f"turboquant/{tag}/scales"]
    assert oracle.golden_digest(TurboQuantCodec.decode(blk)) == DIGESTS[f"turboquant/{tag}/decoded"]


@pytest.mark.parametrize("n", [32, 64, 128, 256])
@pytest.mark.parametrize("bits,qjl,rbits", [(2, False, 1), (3, False, 1), (4, False, 1), (8, False, 1), (4, True, 1), (3, True, 2), (4, True, 3), (8, True, 4)])
def test_codec_bit_exact_against_the_restatement(gpu, n, bits, qjl, rbits):
    from oracle import turboquant as T
    from skainet_b200.kvstore import TurboQuantCodec, TurboQuantConfig
    rng = np.random.default_rng(n * 10 + bits + rbits)
    for trial, seed in enumerate([0, 7, -5, 2147483647, -2147483648]):
        x = (rng.standard_normal(n) * (0.01 if trial == 1 else 2.0)).astype(np.float32)
        if trial == 2:
            x[: n // 2] = 0.0                       # an all-zero group: scale 0, codes 0
        ref = T.encode(x, bits, qjl, rbits, seed)
        got = TurboQuantCodec.encode(x, TurboQuantConfig(bits, qjl, rbits, seed))
        np.testing.assert_array_equal(got["packedCodes"], ref.packed)
        np.testing.assert_array_equal(got["scales"].view(np.uint32), ref.scales.view(np.uint32))
        if qjl:
            np.testing.assert_array_equal(got["residual"][0], ref.residual[0])
            assert np.float32(got["residual"][1]).view(np.uint32) == np.float32(ref.residual[1]).view(np.uint32)
        np.testing.assert_array_equal(TurboQuantCodec.decode(got).view(np.uint32), T.decode(ref).view(np.uint32))
    with pytest.raises(ValueError):
        TurboQuantCodec.encode(np.zeros(100, np.float32), TurboQuantConfig(4))


def test_store_matches_the_restated_store_and_attends_the_decoded_window(gpu, cuda_lib):
    """appendToken / readKeys / readValues / evict / clear / memory accounting as TurboQuantKvCacheStoreTest.kt exercises them,
    keys 4-bit + 1-bit residual, values 3-bit; then one decode step of attention over a window of the store."""
    from oracle import turboquant as T
    from oracle.kv_store import windowed_decode_step
    from skainet_b200.kvstore import DeviceKvCacheStore, TurboQuantConfig
    Lr, H, D, S = 2, 2, 64, 6
    dev = DeviceKvCacheStore(Lr, H, D, S, keyConfig=TurboQuantConfig.polarPlusQjl(4, 1), valueConfig=TurboQuantConfig.polarOnly(3))
    cpu = T.CpuTurboQuantKvStore(Lr, H, D, S, key_cfg=(4, True, 1), value_cfg=(3, False, 1))
    rng = np.random.default_rng(3)
    for pos in range(5):
        for layer in range(Lr):
            k, v = rng.standard_normal((H, D)).astype(np.float32), rng.standard_normal((H, D)).astype(np.float32)
            dev.appendToken(layer, k, v); cpu.append(layer, k, v)
        assert dev.currentSeqLen == cpu.cur == pos + 1
    for layer in range(Lr):
        np.testing.assert_array_equal(dev.readKeys(layer, 0, 5).view(np.uint32), cpu.read_keys(layer, 0, 5).view(np.uint32))
        np.testing.assert_array_equal(dev.readValues(layer, 1, 4).view(np.uint32), cpu.read_values(layer, 1, 4).view(np.uint32))
    assert dev.physicalBytes == sum(cpu.physical_bytes())
    # attention of 4 query heads (2 per cache head) over positions [1, 5)
    q = rng.standard_normal((2 * H, D)).astype(np.float32)
    dq, dout = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer(q.nbytes)
    dev.decodeStep(1, dq.ptr, dout.ptr, 2 * H, 1, 5)
    keys, vals = cpu.read_keys(1, 1, 5), cpu.read_values(1, 1, 5)
    h16 = lambda a: a.astype(np.float16).astype(np.float32)          # head_dim 64, two query heads per cache head: the binary16 route
    ref = windowed_decode_step(q, np.repeat(h16(keys), 2, axis=0), np.repeat(h16(vals), 2, axis=0))
    rel_err_ok(dout.download(np.float32, q.size).reshape(2 * H, D), ref)
    # a full cache refuses the append; evict rolls back; clear empties
    for layer in range(Lr):
        dev.appendToken(layer, q[:H], q[H:]); cpu.append(layer, q[:H], q[H:])
    with pytest.raises(ValueError, match="KV cache is full"):
        dev.appendToken(0, q[:H], q[H:])
    dev.evict(2); cpu.evict(2)
    assert dev.currentSeqLen == 2
    with pytest.raises(ValueError):
        dev.readKeys(0, 0, 3)
    np.testing.assert_array_equal(dev.readKeys(0, 0, 2).view(np.uint32), cpu.read_keys(0, 0, 2).view(np.uint32))
    dev.clear()
    assert dev.currentSeqLen == 0 and dev.physicalBytes == 0
    assert cuda_lib.skainet_cuda_device_status() == 0
    dev.free()


def test_attention_fp32_route_for_other_head_sizes(gpu):
    """head_dim 32 (and group sizes outside 1, 2, 4, 8) are attended in fp32 over the fp32 rows a read returns."""
    from oracle import turboquant as T
    from oracle.kv_store import windowed_decode_step
    from skainet_b200.kvstore import DeviceKvCacheStore, TurboQuantConfig
    H, D, S = 3, 32, 40
    dev = DeviceKvCacheStore(1, H, D, S, keyConfig=TurboQuantConfig.polarOnly(8), valueConfig=TurboQuantConfig.polarPlusQjl(4, 2))
    rng = np.random.default_rng(5)
    for p in range(S):
        dev.appendToken(0, rng.standard_normal((H, D)).astype(np.float32), rng.standard_normal((H, D)).astype(np.float32))
    q = rng.standard_normal((3 * H, D)).astype(np.float32)          # three query heads per cache head
    dq, dout = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer(q.nbytes)
    dev.decodeStep(0, dq.ptr, dout.ptr, 3 * H, 5, S)
    keys, vals = dev.readKeys(0, 5, S), dev.readValues(0, 5, S)
    rel_err_ok(dout.download(np.float32, q.size).reshape(3 * H, D), windowed_decode_step(q, np.repeat(keys, 3, axis=0), np.repeat(vals, 3, axis=0)))
    dev.free()


def test_store_at_decoder_sizes(gpu):
    """8 heads x 128 over 300 positions (the 70B shape's KV heads), 4-bit keys and values: every block bit-exact against
    the restatement on a sample of positions, attention over the whole window within rel 1e-3."""
    from oracle import turboquant as T
    from oracle.kv_store import windowed_decode_step
    from skainet_b200.kvstore import DeviceKvCacheStore, TurboQuantConfig
    H, D, S = 8, 128, 300
    dev = DeviceKvCacheStore(1, H, D, S, keyConfig=TurboQuantConfig.polarOnly(4), valueConfig=TurboQuantConfig.polarOnly(4))
    rng = np.random.default_rng(11)
    ks, vs = rng.standard_normal((S, H, D)).astype(np.float32), rng.standard_normal((S, H, D)).astype(np.float32)
    for p in range(S):
        dev.appendToken(0, ks[p], vs[p])
    keys, vals = dev.readKeys(0, 0, S), dev.readValues(0, 0, S)
    for p in (0, 1, 17, 150, 299):
        for h in (0, 3, 7):
            seed = T.seed_for(0, h, p)
            np.testing.assert_array_equal(keys[h, p].view(np.uint32), T.decode(T.encode(ks[p, h], 4, False, 1, seed)).view(np.uint32))
            np.testing.assert_array_equal(vals[h, p].view(np.uint32),
                                          T.decode(T.encode(vs[p, h], 4, False, 1, T._i32(seed ^ 0x5A5A5A5A))).view(np.uint32))
    err = float(np.sqrt(np.mean((keys - ks.transpose(1, 0, 2)) ** 2)))
    assert 0.02 < err < 0.2            # 4-bit: lossy, but a reconstruction of the input
    q = rng.standard_normal((H, D)).astype(np.float32)
    dq, dout = gpu.DeviceBuffer.from_host(q), gpu.DeviceBuffer(q.nbytes)
    dev.decodeStep(0, dq.ptr, dout.ptr, H, 0, S)
    got = dout.download(np.float32, q.size).reshape(H, D)
    # head_dim 128 with one query head per cache head takes the binary16 route: the decoded rows are rounded to binary16 (as the
    # binary16 store rounds every row it holds) and attended by the split-K kernel
    h16 = lambda a: a.astype(np.float16).astype(np.float32)
    rel_err_ok(got, windowed_decode_step(q, h16(keys), h16(vals)))
    rel_err_ok(got, windowed_decode_step(q, keys, vals), 4e-3)          # and stays close to the unrounded fp32 attention
    dev.free()
