"""The TurboQuant restatement (oracle/turboquant.py) against the digests the reference's own golden test records
(TurboQuantGoldenTest.kt:15-22, Goldens.kt:62-71), plus the codec / packer / store properties the reference tests
(TurboQuantCodecTest.kt, TurboQuantKvCacheStoreTest.kt): CPU only."""
import json
import os

import numpy as np
import pytest

from oracle import ref as R
from oracle import turboquant as T

HERE = os.path.dirname(os.path.abspath(__file__))
DIGESTS = json.load(open(os.path.join(HERE, "golden", "reference_digests.json")))


def byte_digest(b: np.ndarray) -> str:
    b = np.asarray(b, np.uint8)
    return f"n={b.size} fnv={R.fnv1a64(b.tobytes()):016x} head=" + "".join(f"{int(x):02x}" for x in b[:8])


@pytest.mark.parametrize("tag,cfg", [("polar4", dict(bits=4, seed=7)), ("polar3", dict(bits=3, seed=7)),
                                     ("polar4-qjl1", dict(bits=4, use_qjl=True, residual_bits=1, seed=7))])
def test_reference_golden_digests(tag, cfg):
    x = R.golden_floats(128, 0x5EED0003, 3.0)
    blk = T.encode(x, **cfg)
    assert byte_digest(blk.packed) == DIGESTS[f"turboquant/{tag}/codes"]
    assert R.golden_digest(blk.scales) == DIGESTS[f"turboquant/{tag}/scales"]
    assert R.golden_digest(T.decode(blk)) == DIGESTS[f"turboquant/{tag}/decoded"]


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_bit_packer_round_trip_and_sizes(bits):
    rng = np.random.default_rng(bits)
    mc = (1 << (bits - 1)) - 1
    for n in (1, 7, 8, 31, 64, 129):
        codes = rng.integers(-mc, mc + 1, size=n).astype(np.int8)
        p = T.pack(codes, bits)
        assert p.size == T.packed_size(n, bits)
        np.testing.assert_array_equal(T.unpack(p, n, bits), codes)


def test_rotation_is_orthogonal_and_seeded():
    x = np.random.default_rng(0).standard_normal(128).astype(np.float32)
    r = T.rotate(x, 1234)
    assert abs(float(np.linalg.norm(r)) - float(np.linalg.norm(x))) < 1e-4 * float(np.linalg.norm(x))
    np.testing.assert_allclose(T.inverse_rotate(r, 1234), x, atol=2e-6)
    assert not np.array_equal(T.rotate(x, 1235), r)
    y = np.arange(100, dtype=np.float32)            # not a power of two: elements 64.. only get their sign flipped
    ry = T.rotate(y, 5)
    np.testing.assert_array_equal(np.abs(ry[64:]), y[64:])


def test_codec_error_shrinks_with_bits_and_sizes_match_the_formula():
    x = np.random.default_rng(3).standard_normal(128).astype(np.float32)
    errs = []
    for bits in (2, 3, 4, 8):
        b = T.encode(x, bits=bits, seed=11)
        assert b.size_in_bytes == T.encoded_size(128, bits, False, 1)
        errs.append(float(np.sqrt(np.mean((T.decode(b) - x) ** 2))))
    assert errs[0] > errs[1] > errs[2] > errs[3]
    assert errs[3] < 0.02
    q = T.encode(x, bits=4, use_qjl=True, residual_bits=2, seed=11)
    # the block's own accounting leaves out the residual's 4-byte scale that encodedSize counts (TurboQuantCodec.kt:92-98,145-146)
    assert q.size_in_bytes == T.encoded_size(128, 4, True, 2) - 4
    assert np.array_equal(T.decode(T.encode(np.zeros(64, np.float32), seed=3)), np.zeros(64, np.float32))


def test_seed_for_and_kv_store_semantics():
    assert T.seed_for(0, 0, 0) == 0 and T.seed_for(1, 2, 3) != T.seed_for(1, 3, 2)
    st = T.CpuTurboQuantKvStore(2, 2, 64, 4, key_cfg=(4, False, 1), value_cfg=(3, False, 1))
    rng = np.random.default_rng(1)
    toks = [(rng.standard_normal((2, 64)).astype(np.float32), rng.standard_normal((2, 64)).astype(np.float32)) for _ in range(3)]
    for k, v in toks:
        before = st.cur
        st.append(0, k, v)
        assert st.cur == before                      # the length advances with the last layer only
        st.append(1, k * 2, v * 2)
        assert st.cur == before + 1
    assert st.cur == 3
    keys = st.read_keys(0, 0, 3)
    assert keys.shape == (2, 3, 64)
    for p, (k, v) in enumerate(toks):
        for h in range(2):
            np.testing.assert_array_equal(keys[h, p], T.decode(T.encode(k[h], 4, False, 1, T.seed_for(0, h, p))))
            np.testing.assert_array_equal(st.read_values(1, p, p + 1)[h, 0],
                                          T.decode(T.encode(2 * v[h], 3, False, 1, T._i32(T.seed_for(1, h, p) ^ 0x5A5A5A5A))))
    kb, vb = st.physical_bytes()
    assert kb == 2 * 3 * 2 * T.encoded_size(64, 4, False, 1) and vb == 2 * 3 * 2 * T.encoded_size(64, 3, False, 1)
    st.append(0, *toks[0]); st.append(1, *toks[0])
    with pytest.raises(RuntimeError):
        st.append(0, *toks[0])
    st.evict(1)
    assert st.cur == 1
    with pytest.raises(ValueError):
        st.read_keys(0, 0, 2)
    st.clear()
    assert st.cur == 0
