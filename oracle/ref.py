"""CPU oracle for the packed-quantized decode path — TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the bench's CPU-baseline / reference arm may import this module;
the product (``skainet_b200``) never does.

Two checkers live behind it:

* ``port()``  — ``oracle/port.c`` compiled strict-fp32 (``make -C oracle port``): the restatement,
  pinned bit-for-bit to the digests recorded by the reference's golden tests
  (skainet-backends/skainet-backend-cpu/src/goldenTest/kotlin/sk/ainet/exec/golden/Goldens.kt).
* ``ref()``   — the reference's own C kernels compiled unmodified into ``oracle/_ref`` (``make -C
  oracle ref``; only possible where the reference tree is present, the binary travels afterwards).

Also here: the seeded generators the reference's golden tests use (xorshift64*, block builder,
FNV-1a digests — GoldenSupport.kt:18-112), the Q8_0 quantizer rule
(skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/data/Q8_0Quantizer.kt:28-53)
and a Q4_K packer of our own (the reference has none:
skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/data/Requantizers.kt:21-27).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from functools import lru_cache

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "liboracle_port.so")
REF_SO = os.path.join(HERE, "_ref", "libskainet_kernels.so")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)


def build(quiet: bool = True) -> None:
    """Compile the port, and the reference library when the reference tree is present."""
    out = subprocess.run(["make", "-C", HERE, "all"], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(_f32p)


def _bp(a: np.ndarray):
    return a.ctypes.data_as(_u8p)


@lru_cache(maxsize=1)
def port() -> C.CDLL:
    if not os.path.exists(PORT_SO) or os.path.getmtime(PORT_SO) < os.path.getmtime(os.path.join(HERE, "port.c")):
        build()
    lib = C.CDLL(PORT_SO)
    lib.oracle_half_to_float.restype = C.c_float
    lib.oracle_half_to_float.argtypes = [C.c_uint16]
    lib.oracle_float_to_half.restype = C.c_uint16
    lib.oracle_float_to_half.argtypes = [C.c_float]
    lib.oracle_q8_quantize_block.restype = C.c_float
    lib.oracle_argmax.restype = C.c_int32
    lib.oracle_sdpa.restype = None
    lib.oracle_sdpa.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int32] * 6 + [C.c_float] + [C.c_int32] * 3 + \
        [_i32p, _f32p] + [C.c_int32] * 4
    return lib


@lru_cache(maxsize=1)
def ref():
    """The reference's compiled C kernels, or None when no binary is available."""
    if not os.path.exists(REF_SO):
        try:
            build()
        except Exception:
            return None
    if not os.path.exists(REF_SO):
        return None
    lib = C.CDLL(REF_SO)
    for name in ("skainet_q4k_matmul", "skainet_q4k_matmul_rm", "skainet_q8_0_matmul", "skainet_q8_0_matmul_rm"):
        getattr(lib, name).restype = None
        getattr(lib, name).argtypes = [_f32p, C.c_int32, _u8p, C.c_int32, C.c_int32, C.c_int32, _f32p, C.c_int32]
    lib.skainet_f32_rms_norm.restype = None
    lib.skainet_f32_rms_norm.argtypes = [_f32p, _f32p, _f32p, C.c_int32, C.c_int32, C.c_float]
    lib.skainet_f32_sdpa.restype = None
    lib.skainet_f32_sdpa.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int32] * 6 + [C.c_float] + [C.c_int32] * 3 + \
        [_i32p, _f32p] + [C.c_int32] * 4
    lib.skainet_f32_unary.restype = None
    lib.skainet_f32_unary.argtypes = [C.c_int32, _f32p, _f32p, C.c_int32]
    lib.skainet_f32_binary.restype = None
    lib.skainet_f32_binary.argtypes = [C.c_int32, _f32p, C.c_int32, _f32p, C.c_int32, _f32p, C.c_int32, C.c_int32]
    lib.skainet_smoke_double.restype = None
    lib.skainet_smoke_double.argtypes = [_f32p, _f32p, C.c_int32]
    return lib


# --------------------------------------------------------------------------------------------------
# Seeded generators and digests of the reference's golden tests (GoldenSupport.kt)
# --------------------------------------------------------------------------------------------------
_M64 = (1 << 64) - 1


class GoldenRng:
    """xorshift64* exactly as GoldenSupport.kt:18-31."""

    def __init__(self, seed: int):
        self.s = (seed & _M64) or 0x9E3779B97F4A7C15

    def next_long(self) -> int:
        x = self.s
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.s = x
        return (x * 0x2545F4914F6CDD1D) & _M64

    def next_byte(self) -> int:
        return self.next_long() >> 56

    def next_float(self) -> np.float32:
        return np.float32(((self.next_long() >> 40) & 0xFFFFFF) / 16777216.0)

    def next_signed(self) -> np.float32:
        return np.float32(self.next_float() * np.float32(2.0) - np.float32(1.0))


def golden_half(v: np.float32) -> int:
    """The golden tests' fp32->fp16: mantissa TRUNCATED, subnormals flushed (GoldenSupport.kt:34-43)."""
    bits = int(np.float32(v).view(np.uint32))
    sign = (bits >> 16) & 0x8000
    expo = ((bits >> 23) & 0xFF) - 127 + 15
    mant = bits & 0x7FFFFF
    if expo <= 0:
        return sign
    if expo >= 31:
        return sign | 0x7C00
    return sign | (expo << 10) | (mant >> 13)


GOLDEN_GEOMETRY = {"Q8_0": (32, 34), "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210)}


def golden_block(enc: str, rng: GoldenRng) -> bytes:
    """A random but valid block (GoldenSupport.kt:49-69): d, dMin and m are drawn for every encoding."""
    _, nbytes = GOLDEN_GEOMETRY[enc]
    b = bytearray(rng.next_byte() for _ in range(nbytes))
    d = np.float32(rng.next_float() * np.float32(0.045) + np.float32(0.005))
    dmin = np.float32(rng.next_float() * np.float32(0.02) + np.float32(0.005))
    _m = rng.next_signed() * np.float32(0.5)
    def le16(off, h):
        b[off] = h & 0xFF
        b[off + 1] = (h >> 8) & 0xFF
    if enc == "Q8_0":
        le16(0, golden_half(d))
    elif enc in ("Q4_K", "Q5_K"):
        le16(0, golden_half(d))
        le16(2, golden_half(dmin))
    elif enc == "Q6_K":
        le16(208, golden_half(d))
    return bytes(b)


def golden_weight_blocks(enc: str, rows: int, blocks_per_row: int, seed: int):
    rng = GoldenRng(seed)
    return [[golden_block(enc, rng) for _ in range(blocks_per_row)] for _ in range(rows)]


def golden_row_major(blocks) -> np.ndarray:
    return np.frombuffer(b"".join(b"".join(r) for r in blocks), dtype=np.uint8).copy()


def golden_block_major(blocks) -> np.ndarray:
    rows, per = len(blocks), len(blocks[0])
    return np.frombuffer(b"".join(blocks[o][bi] for bi in range(per) for o in range(rows)), dtype=np.uint8).copy()


def golden_floats(n: int, seed: int, scale: float = 1.0) -> np.ndarray:
    rng = GoldenRng(seed)
    return np.array([rng.next_signed() * np.float32(scale) for _ in range(n)], dtype=np.float32)


def fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for byte in data:
        h = ((h ^ byte) * 1099511628211) & _M64
    return h


def golden_digest(values: np.ndarray) -> str:
    """GoldenSupport.digest(FloatArray): FNV-1a-64 over little-endian float bits + first four patterns."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    bits = v.view(np.uint32)
    head = ",".join(f"{int(x):08x}" for x in bits[:4])
    return f"n={v.size} fnv={fnv1a64(v.astype('<f4').tobytes()):016x} head={head}"


# --------------------------------------------------------------------------------------------------
# Quantizers (host side, numpy)
# --------------------------------------------------------------------------------------------------
def quantize_q8_0(values: np.ndarray) -> np.ndarray:
    """fp32 -> packed Q8_0 bytes, the rule of Q8_0Quantizer.kt:28-53: d = amax/127 (fp32), id = 1/d,
    code = roundToInt(x*id) (half up) clamped to +-127, stored scale = RNE fp16 of d."""
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(v).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    q = np.floor((v * inv[:, None]).astype(np.float32).astype(np.float64) + 0.5)
    q = np.clip(q, -127, 127).astype(np.int8)
    out = np.empty((v.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def pack_k4_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of ggml get_scale_min_k4: [n,8] 6-bit scales and mins -> [n,12] bytes."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros((sc.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = (sc[:, 0:4] & 0x3F) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 0x3F) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return out


def quantize_q4k(values: np.ndarray) -> np.ndarray:
    """fp32 -> packed Q4_K bytes (144 B per 256 values). Our own min/max packer; any valid packer
    serves, because every comparison is made on identical packed bytes."""
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 8, 32)
    lo = np.minimum(v.min(axis=2), 0.0)
    hi = np.maximum(v.max(axis=2), lo)
    scale = ((hi - lo) / 15.0).astype(np.float32)
    mins = (-lo).astype(np.float32)
    d = (scale.max(axis=1) / 63.0).astype(np.float16)
    dmin = (mins.max(axis=1) / 63.0).astype(np.float16)
    df = d.astype(np.float32)
    dmf = dmin.astype(np.float32)
    sc = np.where(df[:, None] > 0, np.rint(scale / np.where(df > 0, df, 1)[:, None]), 0).clip(0, 63).astype(np.int32)
    mn = np.where(dmf[:, None] > 0, np.rint(mins / np.where(dmf > 0, dmf, 1)[:, None]), 0).clip(0, 63).astype(np.int32)
    eff = (df[:, None] * sc).astype(np.float32)
    off = (dmf[:, None] * mn).astype(np.float32)
    q = np.where(eff[:, :, None] > 0, np.rint((v + off[:, :, None]) / np.where(eff > 0, eff, 1)[:, :, None]), 0)
    q = q.clip(0, 15).astype(np.uint8)
    out = np.empty((v.shape[0], 144), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = pack_k4_scales(sc, mn)
    qg = q.reshape(-1, 4, 2, 32)  # group, lo/hi sub-block, byte
    out[:, 16:] = (qg[:, :, 0, :] | (qg[:, :, 1, :] << 4)).reshape(-1, 128)
    return out.reshape(-1)


BLOCK_BYTES = {"Q8_0": 34, "Q4_K": 144, "Q5_K": 176, "Q6_K": 210}
BLOCK_ELEMS = {"Q8_0": 32, "Q4_K": 256, "Q5_K": 256, "Q6_K": 256}


def to_feed_order(row_major: np.ndarray, enc: str, rows: int, cols: int) -> np.ndarray:
    """[o][b] blocks -> [b][o] blocks: the relayout of
    skainet-backends/skainet-backend-api/src/commonMain/kotlin/sk/ainet/backend/api/kernel/PackedWeights.kt:63-95."""
    bb, bpr = BLOCK_BYTES[enc], cols // BLOCK_ELEMS[enc]
    return np.ascontiguousarray(row_major.reshape(rows, bpr, bb).transpose(1, 0, 2)).reshape(-1)


# --------------------------------------------------------------------------------------------------
# Function wrappers over the port (and the compiled reference where it exists)
# --------------------------------------------------------------------------------------------------
def dequant(enc: str, packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    nblocks = packed.size // BLOCK_BYTES[enc]
    out = np.empty(nblocks * BLOCK_ELEMS[enc], dtype=np.float32)
    fn = {"Q8_0": "oracle_dequant_q8_0", "Q4_K": "oracle_dequant_q4k", "Q5_K": "oracle_dequant_q5k",
          "Q6_K": "oracle_dequant_q6k"}[enc]
    getattr(port(), fn)(_bp(packed), C.c_int64(nblocks), _fp(out))
    return out


def scalar_matmul(enc: str, x: np.ndarray, w_feed: np.ndarray, input_dim: int, output_dim: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(output_dim, dtype=np.float32)
    fn = {"Q8_0": "oracle_scalar_matmul_q8_0", "Q4_K": "oracle_scalar_matmul_q4k"}[enc]
    getattr(port(), fn)(_fp(x), _bp(w_feed), C.c_int32(input_dim), C.c_int32(output_dim), _fp(out))
    return out


def matmul(enc: str, x: np.ndarray, w: np.ndarray, input_dim: int, output_dim: int, order: str = "rm",
           use_ref: bool = False) -> np.ndarray:
    """x[M, input_dim] (or [input_dim]) times the packed [output_dim, input_dim] weight, the native
    way: one matvec per activation row (PackedViewMatmulKernel.kt:99-107)."""
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, input_dim)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    out = np.zeros((x2.shape[0], output_dim), dtype=np.float32)
    lib = ref() if use_ref else None
    if use_ref and lib is None:
        raise RuntimeError("oracle/_ref is not built")
    if enc in ("Q5_K", "Q6_K") and order != "rm":
        raise ValueError("the Q5_K / Q6_K restatements take the row-major order only")
    for r in range(x2.shape[0]):
        if lib is not None:
            name = {"Q8_0": "skainet_q8_0_matmul", "Q4_K": "skainet_q4k_matmul", "Q5_K": "skainet_q5k_matmul",
                    "Q6_K": "skainet_q6k_matmul"}[enc] + ("_rm" if order == "rm" else "")
            getattr(lib, name)(_fp(x2[r]), 0, _bp(w), 0, input_dim, output_dim, _fp(out[r]), 0)
        elif enc in ("Q5_K", "Q6_K"):
            fn = {"Q5_K": "oracle_q5k_matmul", "Q6_K": "oracle_q6k_matmul"}[enc]
            getattr(port(), fn)(_fp(x2[r]), _bp(w), C.c_int32(input_dim), C.c_int32(output_dim), _fp(out[r]))
        else:
            fn = {"Q8_0": "oracle_q8_0_matmul", "Q4_K": "oracle_q4k_matmul"}[enc]
            getattr(port(), fn)(_fp(x2[r]), _bp(w), C.c_int32(input_dim), C.c_int32(output_dim), _fp(out[r]),
                                C.c_int32(0 if order == "rm" else 1))
    return out.reshape(x.shape[:-1] + (output_dim,)) if x.ndim > 1 else out[0]


def random_kquant_blocks(enc: str, rows: int, cols: int, seed: int = 0) -> np.ndarray:
    """Valid random Q5_K / Q6_K super-blocks [rows * cols/256] in canonical GGUF order: random code bits, small scales,
    f16 d (and dmin) of a magnitude that keeps outputs O(1). Not a quantizer: the matvec tests only need well-formed bytes."""
    rng = np.random.default_rng(seed)
    nb = rows * (cols // 256)
    if enc == "Q6_K":
        blk = rng.integers(0, 256, (nb, 210), dtype=np.uint8)
        blk[:, 192:208] = rng.integers(-48, 48, (nb, 16)).astype(np.int8).view(np.uint8)
        blk[:, 208:210] = np.abs(0.0008 * rng.standard_normal(nb)).astype(np.float16).view(np.uint8).reshape(nb, 2)
        return blk.reshape(-1)
    if enc == "Q5_K":
        blk = rng.integers(0, 256, (nb, 176), dtype=np.uint8)
        blk[:, 0:2] = np.abs(0.0006 * rng.standard_normal(nb)).astype(np.float16).view(np.uint8).reshape(nb, 2)
        blk[:, 2:4] = np.abs(0.004 * rng.standard_normal(nb)).astype(np.float16).view(np.uint8).reshape(nb, 2)
        return blk.reshape(-1)
    raise ValueError(enc)


def q8_quantize(x: np.ndarray):
    """Per-256 int8 activation quantization (q4k_matmul.c:74-92) -> (codes int8[k], d_in float[k/256])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    nb = x.size // 256
    q8 = np.empty(x.size, dtype=np.int8)
    d = np.empty(nb, dtype=np.float32)
    for b in range(nb):
        d[b] = port().oracle_q8_quantize_block(_fp(x[b * 256:]), q8[b * 256:].ctypes.data_as(C.c_void_p))
    return q8, d


def rms_norm(x: np.ndarray, gamma, eps: float, use_ref: bool = False) -> np.ndarray:
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    g = None if gamma is None else np.ascontiguousarray(gamma, dtype=np.float32)
    gp = _fp(g) if g is not None else None
    if use_ref:
        ref().skainet_f32_rms_norm(_fp(x2), gp, _fp(out), x2.shape[0], x2.shape[1], eps)
    else:
        port().oracle_rms_norm(_fp(x2), gp, _fp(out), C.c_int32(x2.shape[0]), C.c_int32(x2.shape[1]), C.c_float(eps))
    return out.reshape(x.shape)


def sdpa(q, k, v, scale, causal=True, window=0, right_context=0, lengths=None, mask=None, use_ref=False):
    """q [B,H,Sq,D], k/v [B,Hkv,Skv,D] fp32 -> out [B,H,Sq,D] (f32_fused.c:304-396)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    B, H, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    out = np.zeros_like(q)
    lp = None
    if lengths is not None:
        lengths = np.ascontiguousarray(lengths, dtype=np.int32)
        lp = lengths.ctypes.data_as(_i32p)
    mp, md = None, (0, 0, 0, 0)
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.float32)
        md = (1,) * (4 - mask.ndim) + tuple(mask.shape)
        mp = _fp(mask)
    args = [_fp(q), _fp(k), _fp(v), _fp(out), B, H, Hkv, Sq, Skv, D, C.c_float(scale), int(causal), window,
            right_context, lp, mp, md[0], md[1], md[2], md[3]]
    if use_ref:
        ref().skainet_f32_sdpa(*args)
    else:
        port().oracle_sdpa(*args)
    return out


def silu(x: np.ndarray, use_ref: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    if use_ref:
        ref().skainet_f32_unary(2, _fp(x.reshape(-1)), _fp(out.reshape(-1)), x.size)
    else:
        port().oracle_silu(_fp(x.reshape(-1)), _fp(out.reshape(-1)), C.c_int32(x.size))
    return out


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(gate)
    port().oracle_swiglu(_fp(gate.reshape(-1)), _fp(up.reshape(-1)), _fp(out.reshape(-1)), C.c_int32(gate.size))
    return out


def rope(x: np.ndarray, heads: int, d: int, pos: int, theta: float = 1e4, mode: int = 0) -> np.ndarray:
    out = np.ascontiguousarray(x, dtype=np.float32).copy()
    port().oracle_rope(_fp(out.reshape(-1)), C.c_int32(heads), C.c_int32(d), C.c_int32(pos), C.c_float(theta),
                       C.c_int32(mode))
    return out


def rope_seq(x: np.ndarray, pos0: int = 0, theta: float = 1e4, mode: int = 0) -> np.ndarray:
    """x [heads, len, d]: row t of every head rotated for position pos0 + t (keys as a decoder caches them)."""
    out = np.ascontiguousarray(x, dtype=np.float32).copy()
    heads, ln, d = out.shape
    port().oracle_rope_seq(_fp(out.reshape(-1)), C.c_int32(heads), C.c_int32(ln), C.c_int32(d), C.c_int32(pos0),
                           C.c_float(theta), C.c_int32(mode))
    return out


def round_f16(x: np.ndarray) -> np.ndarray:
    """fp32 -> binary16 (round to nearest even) -> fp32: what an f16 KV cache holds."""
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def argmax(x: np.ndarray) -> int:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return int(port().oracle_argmax(_fp(x), C.c_int32(x.size)))
