"""CPU restatement of the reference's TurboQuant KV-cache compression. TEST INFRASTRUCTURE ONLY: nothing the product
ships imports this file; tests use it as the checker for the CUDA codec and store.

Follows, function by function (paths inside the reference tree, skainet-lang/skainet-lang-core/src/commonMain/kotlin/
sk/ainet/lang/tensor/):

  ops/turboquant/RandomRotation.kt:38-131   seeded sign flips + normalised Walsh-Hadamard transform, seedFor
  ops/turboquant/ScalarQuantizer.kt:35-73   symmetric per-32 scalar quantizer (fp32 scale = absmax / maxCode)
  ops/turboquant/BitPacker.kt:23-181        2 / 3 / 4 / 8-bit packing with bias 2^(bits-1)
  ops/turboquant/QjlResidual.kt:24-97       1-bit sign residual (rms scale) and 2-4 bit scalar residual (mean scale)
  ops/turboquant/TurboQuantCodec.kt:33-99   encode / decode / encodedSize
  storage/TurboQuantKvCacheStore.kt:62-199  per (layer, position, head) blocks, value seed = key seed xor 0x5A5A5A5A

The sign flips come from `kotlin.random.Random(seed)`, the Kotlin standard library's xorwow generator (Marsaglia 2003):
state (x, y, z, w, v, addend) = (seed, seed >> 31, 0, 0, ~seed, (seed << 10) ^ ((seed >> 31) >>> 4)), 64 draws discarded,
nextBoolean = top bit of the next 32-bit draw. It is restated here from that published algorithm.

Pinned: tests/test_oracle.py reproduces the nine digests the reference's golden test records for this path
(`turboquant/{polar4,polar3,polar4-qjl1}/{codes,scales,decoded}`, skainet-backends/skainet-backend-cpu/src/goldenTest/
kotlin/sk/ainet/exec/golden/Goldens.kt:62-71, inputs of TurboQuantGoldenTest.kt:15-22) bit for bit.

All arithmetic is fp32 with every operation rounded on its own (the JVM does not fuse), in the reference's order.
"""
from __future__ import annotations

import numpy as np

F = np.float32
GROUP = 32
_M32 = 0xFFFFFFFF


def _i32(v: int) -> int:
    v &= _M32
    return v - (1 << 32) if v & 0x80000000 else v


class KotlinRandom:
    """kotlin.random.Random(seed: Int) (XorWowRandom)."""

    def __init__(self, seed: int):
        s1 = seed & _M32
        s2 = (_i32(seed) >> 31) & _M32
        self.x, self.y, self.z, self.w = s1, s2, 0, 0
        self.v = (~s1) & _M32
        self.addend = ((s1 << 10) & _M32) ^ (s2 >> 4)
        for _ in range(64):
            self.next_int()

    def next_int(self) -> int:
        t = self.x
        t ^= t >> 2
        self.x, self.y, self.z = self.y, self.z, self.w
        v0 = self.v
        self.w = v0
        t = (t ^ ((t << 1) & _M32)) ^ v0 ^ ((v0 << 4) & _M32)
        self.v = t
        self.addend = (self.addend + 362437) & _M32
        return (t + self.addend) & _M32

    def next_boolean(self) -> bool:
        return (self.next_int() >> 31) != 0


def sign_bits(seed: int, n: int) -> np.ndarray:
    """True where RandomRotation.randomSignFlip negates the element."""
    rng = KotlinRandom(seed)
    return np.array([rng.next_boolean() for _ in range(n)], dtype=bool)


def seed_for(layer: int, head: int, position: int) -> int:
    """RandomRotation.seedFor: 31-polynomial of the triple through the MurmurHash3 finalizer, as a signed 32-bit int."""
    h = layer & _M32
    h = (h * 31 + head) & _M32
    h = (h * 31 + position) & _M32
    h ^= h >> 16
    h = (h * 0x85EBCA6B) & _M32
    h ^= h >> 13
    h = (h * 0xC2B2AE35) & _M32
    h ^= h >> 16
    return _i32(h)


def walsh_hadamard(v: np.ndarray) -> np.ndarray:
    """In place over the largest power of two <= n, butterflies in the reference's order, then * 1/sqrt(len)."""
    n = v.size
    if n <= 1:
        return v
    ln = 1
    while ln * 2 <= n:
        ln *= 2
    h = 1
    while h < ln:
        a = v[:ln].reshape(-1, 2, h)
        x = a[:, 0, :].copy(); y = a[:, 1, :].copy()
        a[:, 0, :] = (x + y).astype(F); a[:, 1, :] = (x - y).astype(F)
        h *= 2
    norm = F(1.0) / np.sqrt(F(ln))
    v[:ln] = (v[:ln] * norm).astype(F)
    return v


def rotate(v: np.ndarray, seed: int) -> np.ndarray:
    v = np.array(v, dtype=F)
    s = sign_bits(seed, v.size)
    v[s] = -v[s]
    return walsh_hadamard(v)


def inverse_rotate(v: np.ndarray, seed: int) -> np.ndarray:
    v = walsh_hadamard(np.array(v, dtype=F))
    s = sign_bits(seed, v.size)
    v[s] = -v[s]
    return v


def quantize(v: np.ndarray, bits: int):
    """ScalarQuantizer.quantize -> (int8 codes, fp32 scales per 32)."""
    assert bits in (2, 3, 4, 8)
    max_code = (1 << (bits - 1)) - 1
    n = v.size
    ng = (n + GROUP - 1) // GROUP
    codes = np.zeros(n, dtype=np.int8)
    scales = np.zeros(ng, dtype=F)
    for g in range(ng):
        seg = v[g * GROUP:(g + 1) * GROUP].astype(F)
        amax = F(np.max(np.abs(seg))) if seg.size else F(0)
        scale = F(amax / F(max_code)) if amax > 0 else F(0)
        scales[g] = scale
        if scale > 0:
            inv = F(F(1.0) / scale)
            q = np.rint((seg * inv).astype(F)).astype(np.int64)        # kotlin.math.round: ties to even
            codes[g * GROUP:g * GROUP + seg.size] = np.clip(q, -max_code, max_code).astype(np.int8)
    return codes, scales


def dequantize(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    out = np.zeros(codes.size, dtype=F)
    for g in range(scales.size):
        seg = codes[g * GROUP:(g + 1) * GROUP]
        out[g * GROUP:g * GROUP + seg.size] = (seg.astype(F) * scales[g]).astype(F)
    return out


def packed_size(count: int, bits: int) -> int:
    return {2: (count + 3) // 4, 3: (count * 3 + 7) // 8, 4: (count + 1) // 2, 8: count}[bits]


def pack(codes: np.ndarray, bits: int) -> np.ndarray:
    n = codes.size
    out = np.zeros(packed_size(n, bits), dtype=np.uint8)
    if bits == 8:
        return codes.astype(np.int8).view(np.uint8).copy()
    bias = 1 << (bits - 1)
    mask = (1 << bits) - 1
    u = (codes.astype(np.int32) + bias) & mask
    if bits == 2:
        for i in range(n):
            out[i // 4] |= np.uint8(u[i] << ((i % 4) * 2))
    elif bits == 4:
        for i in range(n):
            out[i // 2] |= np.uint8(u[i] << (4 * (i % 2)))
    else:   # 3 bits: a little-endian bit stream
        pos = 0
        for i in range(n):
            b, o = pos // 8, pos % 8
            out[b] |= np.uint8((int(u[i]) << o) & 0xFF)
            if o > 5 and b + 1 < out.size:
                out[b + 1] |= np.uint8(int(u[i]) >> (8 - o))
            pos += 3
    return out


def unpack(packed: np.ndarray, count: int, bits: int) -> np.ndarray:
    if bits == 8:
        return packed[:count].view(np.int8).copy()
    bias = 1 << (bits - 1)
    out = np.zeros(count, dtype=np.int8)
    if bits == 2:
        for i in range(count):
            out[i] = ((int(packed[i // 4]) >> ((i % 4) * 2)) & 3) - bias
    elif bits == 4:
        for i in range(count):
            out[i] = ((int(packed[i // 2]) >> (4 * (i % 2))) & 15) - bias
    else:
        pos = 0
        for i in range(count):
            b, o = pos // 8, pos % 8
            val = (int(packed[b]) >> o) & 7
            if o > 5 and b + 1 < packed.size:
                first = 8 - o
                val = ((int(packed[b]) >> o) & ((1 << first) - 1)) | ((int(packed[b + 1]) & ((1 << (3 - first)) - 1)) << first)
            out[i] = val - bias
            pos += 3
    return out


def _seq_sum_sq(v: np.ndarray) -> np.float32:
    s = F(0)
    for x in v.astype(F):
        s = F(s + F(x * x))
    return s


def residual_encode(res: np.ndarray, residual_bits: int, seed: int):
    """QjlResidual.encode -> (packed bytes, fp32 scale)."""
    dim = res.size
    if residual_bits == 1:
        scale = F(np.sqrt(F(_seq_sum_sq(res) / F(dim))))
        s = sign_bits(seed, dim)                      # True -> +1, False -> -1
        packed = np.zeros((dim + 7) // 8, dtype=np.uint8)
        for i in range(dim):
            sg = F(1.0) if s[i] else F(-1.0)
            if F(res[i] * sg) >= 0:
                packed[i // 8] |= np.uint8(1 << (i % 8))
        return packed, scale
    codes, scales = quantize(res, residual_bits)
    mean = F(0)
    for sc in scales:
        mean = F(mean + sc)
    mean = F(mean / F(scales.size)) if scales.size else F(0)
    return pack(codes, residual_bits), mean


def residual_decode_into(packed: np.ndarray, scale, residual_bits: int, dim: int, out: np.ndarray, seed: int) -> None:
    if residual_bits == 1:
        s = sign_bits(seed, dim)
        for i in range(dim):
            sg = F(1.0) if s[i] else F(-1.0)
            val = F(scale) if (int(packed[i // 8]) >> (i % 8)) & 1 else F(-F(scale))
            out[i] = F(out[i] + F(val * sg))
    else:
        codes = unpack(packed, dim, residual_bits)
        for i in range(dim):
            out[i] = F(out[i] + F(F(codes[i]) * F(scale)))


class Block:
    """TurboQuantBlock."""

    def __init__(self, packed, scales, seed, bits, n, residual=None, residual_bits=0):
        self.packed, self.scales, self.seed, self.bits, self.n = packed, scales, seed, bits, n
        self.residual, self.residual_bits = residual, residual_bits       # residual = (packed, scale) or None

    @property
    def size_in_bytes(self) -> int:
        return self.packed.size + self.scales.size * 4 + 4 + (self.residual[0].size if self.residual else 0)


def encode(v: np.ndarray, bits: int = 4, use_qjl: bool = False, residual_bits: int = 1, seed: int = 0) -> Block:
    rot = rotate(v, seed)
    codes, scales = quantize(rot, bits)
    residual = None
    if use_qjl:
        deq = dequantize(codes, scales)
        residual = residual_encode((rot - deq).astype(F), residual_bits, _i32(seed + 1))
    return Block(pack(codes, bits), scales, seed, bits, v.size, residual, residual_bits if use_qjl else 0)


def decode(b: Block) -> np.ndarray:
    out = dequantize(unpack(b.packed, b.n, b.bits), b.scales)
    if b.residual is not None:
        residual_decode_into(b.residual[0], b.residual[1], b.residual_bits, b.n, out, _i32(b.seed + 1))
    return inverse_rotate(out, b.seed)


def encoded_size(n: int, bits: int, use_qjl: bool, residual_bits: int) -> int:
    return packed_size(n, bits) + ((n + GROUP - 1) // GROUP) * 4 + 4 + ((packed_size(n, residual_bits) + 4) if use_qjl else 0)


class CpuTurboQuantKvStore:
    """TurboQuantKvCacheStore: one block per (layer, position, head) for keys and for values."""

    def __init__(self, n_layers, n_heads, head_dim, max_seq, key_cfg=(4, False, 1), value_cfg=(4, False, 1)):
        self.L, self.H, self.D, self.S = n_layers, n_heads, head_dim, max_seq
        self.key_cfg, self.value_cfg = key_cfg, value_cfg
        self.cur = 0
        self.k = [[[None] * n_heads for _ in range(max_seq)] for _ in range(n_layers)]
        self.v = [[[None] * n_heads for _ in range(max_seq)] for _ in range(n_layers)]

    def append(self, layer: int, key: np.ndarray, value: np.ndarray) -> None:
        if not 0 <= layer < self.L:
            raise ValueError("layer out of range")
        if self.cur >= self.S:
            raise RuntimeError("KV cache is full")
        key = np.asarray(key, F).reshape(self.H, self.D); value = np.asarray(value, F).reshape(self.H, self.D)
        pos = self.cur
        for h in range(self.H):
            ks = seed_for(layer, h, pos)
            vs = _i32(ks ^ 0x5A5A5A5A)
            self.k[layer][pos][h] = encode(key[h], self.key_cfg[0], self.key_cfg[1], self.key_cfg[2], ks)
            self.v[layer][pos][h] = encode(value[h], self.value_cfg[0], self.value_cfg[1], self.value_cfg[2], vs)
        if layer == self.L - 1:
            self.cur += 1

    def _read(self, blocks, layer, start, end) -> np.ndarray:
        if not 0 <= layer < self.L or not 0 <= start <= end or end > self.cur:
            raise ValueError("bad range")
        out = np.zeros((self.H, end - start, self.D), F)
        for h in range(self.H):
            for p in range(start, end):
                out[h, p - start] = decode(blocks[layer][p][h])
        return out

    def read_keys(self, layer, start, end):
        return self._read(self.k, layer, start, end)

    def read_values(self, layer, start, end):
        return self._read(self.v, layer, start, end)

    def evict(self, from_pos: int) -> None:
        if not 0 <= from_pos <= self.cur:
            raise ValueError("evict out of range")
        for l in range(self.L):
            for p in range(from_pos, self.S):
                self.k[l][p] = [None] * self.H; self.v[l][p] = [None] * self.H
        self.cur = from_pos

    def clear(self) -> None:
        self.evict(0)

    def physical_bytes(self):
        kb = sum(b.size_in_bytes for l in range(self.L) for p in range(self.cur) for b in self.k[l][p] if b is not None)
        vb = sum(b.size_in_bytes for l in range(self.L) for p in range(self.cur) for b in self.v[l][p] if b is not None)
        return kb, vb
