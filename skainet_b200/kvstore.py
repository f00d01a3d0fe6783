"""Host-side handle of the device KV-cache store (include/skainet_cuda.h, section 3): the mirror of the reference's
KvCacheStore interface — appendToken / readKeys / readValues / evict / clear / currentSeqLen / windowStart
(skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/KvCacheStore.kt:125-157,
DefaultKvCacheStore.kt:30-36,170-177) — with the cache resident in HBM as binary16 and attention reading it in place."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


class TurboQuantConfig:
    """TurboQuantConfig of the reference (TurboQuantCodec.kt:104-131): bits in {2,3,4,8}; useQjl adds the residual stage."""

    def __init__(self, bits: int = 4, useQjl: bool = False, residualBits: int = 1, seed: int = 0):
        if bits not in (2, 3, 4, 8):
            raise ValueError(f"bits must be 2, 3, 4, or 8, got {bits}")
        if useQjl and not 1 <= residualBits <= 4:
            raise ValueError(f"residualBits must be 1-4, got {residualBits}")
        self.bits, self.useQjl, self.residualBits, self.seed = bits, useQjl, residualBits, seed

    @classmethod
    def polarOnly(cls, bits: int = 4, seed: int = 0) -> "TurboQuantConfig":
        return cls(bits, False, 1, seed)

    @classmethod
    def polarPlusQjl(cls, bits: int = 4, residualBits: int = 1, seed: int = 0) -> "TurboQuantConfig":
        return cls(bits, True, residualBits, seed)

    @property
    def rbits(self) -> int:
        return self.residualBits if self.useQjl else 0


def packed_size(count: int, bits: int) -> int:
    """Bytes of `count` packed codes (BitPacker.kt:46-54); one bit per element for the 1-bit residual (QjlResidual.kt:36)."""
    return {1: (count + 7) // 8, 2: (count + 3) // 4, 3: (count * 3 + 7) // 8, 4: (count + 1) // 2, 8: count}[bits]


class TurboQuantCodec:
    """TurboQuantCodec.encode / decode (TurboQuantCodec.kt:33-85) on the GPU, one vector of 32 / 64 / 128 / 256 floats per call."""

    @staticmethod
    def encode(x: np.ndarray, config: TurboQuantConfig) -> dict:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        n, rb = x.size, config.rbits
        codes = np.zeros(packed_size(n, config.bits) if n in (32, 64, 128, 256) else 1, np.uint8)
        scales = np.zeros(max(1, n // 32), np.float32)
        resid = np.zeros(packed_size(n, rb) if rb else 1, np.uint8)
        rscale = C.c_float(0.0)
        L.check(L.lib().skainet_cuda_turboquant_encode(x.ctypes.data_as(L.f32p), n, config.bits, rb, config.seed, codes.ctypes.data_as(L.u8p),
                                                       scales.ctypes.data_as(L.f32p), resid.ctypes.data_as(L.u8p), C.byref(rscale)))
        return {"packedCodes": codes, "scales": scales, "seed": config.seed, "bits": config.bits, "elementCount": n,
                "residual": (resid, float(rscale.value), rb) if rb else None}

    @staticmethod
    def decode(block: dict) -> np.ndarray:
        n = block["elementCount"]
        out = np.empty(n, np.float32)
        resid, rscale, rb = block["residual"] if block["residual"] else (np.zeros(1, np.uint8), 0.0, 0)
        L.check(L.lib().skainet_cuda_turboquant_decode(block["packedCodes"].ctypes.data_as(L.u8p), block["scales"].ctypes.data_as(L.f32p),
                                                       resid.ctypes.data_as(L.u8p), C.c_float(rscale), n, block["bits"], rb, block["seed"],
                                                       out.ctypes.data_as(L.f32p)))
        return out


class DeviceKvCacheStore:
    def __init__(self, numLayers: int, numHeads: int, headDim: int, maxSeqLen: int, slidingWindow: bool = False,
                 keyConfig: TurboQuantConfig | None = None, valueConfig: TurboQuantConfig | None = None):
        """keyConfig / valueConfig given: a TurboQuant store (the mirror of TurboQuantKvCacheStore), else binary16 rows."""
        h = C.c_int64()
        if (keyConfig is None) != (valueConfig is None):
            raise ValueError("a TurboQuant store takes both a key and a value configuration")
        if keyConfig is not None:
            if slidingWindow:
                raise ValueError("the TurboQuant store has no sliding-window mode")
            L.check(L.lib().skainet_cuda_kv_create_turboquant(numLayers, numHeads, headDim, maxSeqLen, keyConfig.bits, keyConfig.rbits,
                                                              valueConfig.bits, valueConfig.rbits, C.byref(h)))
        else:
            L.check(L.lib().skainet_cuda_kv_create(numLayers, numHeads, headDim, maxSeqLen, 1 if slidingWindow else 0, C.byref(h)))
        self.handle = h.value
        self.numLayers, self.numHeads, self.headDim, self.maxSeqLen, self.slidingWindow = numLayers, numHeads, headDim, maxSeqLen, slidingWindow

    def _info(self):
        out = (C.c_int64 * 8)()
        L.check(L.lib().skainet_cuda_kv_info(self.handle, out))
        return list(out)

    @property
    def currentSeqLen(self) -> int:
        return int(self._info()[0])

    @property
    def windowStart(self) -> int:
        return int(self._info()[1])

    @property
    def physicalBytes(self) -> int:
        return int(self._info()[7])

    def appendToken(self, layer: int, key: np.ndarray, value: np.ndarray) -> None:
        k = np.ascontiguousarray(key, dtype=np.float32).reshape(-1)
        v = np.ascontiguousarray(value, dtype=np.float32).reshape(-1)
        n = self.numHeads * self.headDim
        if k.size != n:
            raise ValueError(f"Key size mismatch: expected {n}, got {k.size}")
        if v.size != n:
            raise ValueError(f"Value size mismatch: expected {n}, got {v.size}")
        L.check(L.lib().skainet_cuda_kv_append(self.handle, layer, k.ctypes.data_as(L.f32p), v.ctypes.data_as(L.f32p)))

    def appendTokenDevice(self, layer: int, key_ptr: int, value_ptr: int, stream: int = 0) -> None:
        L.check(L.lib().skainet_cuda_kv_append_dev(self.handle, layer, key_ptr, value_ptr, stream))

    def _read(self, which: int, layer: int, startPos: int, endPos: int | None) -> np.ndarray:
        end = self.currentSeqLen if endPos is None else endPos
        out = np.empty((self.numHeads, max(0, end - startPos), self.headDim), dtype=np.float32)
        L.check(L.lib().skainet_cuda_kv_read(self.handle, layer, which, startPos, end, out.ctypes.data_as(L.f32p)))
        return out

    def readKeys(self, layer: int, startPos: int = 0, endPos: int | None = None) -> np.ndarray:
        return self._read(0, layer, startPos, endPos)

    def readValues(self, layer: int, startPos: int = 0, endPos: int | None = None) -> np.ndarray:
        return self._read(1, layer, startPos, endPos)

    def evict(self, fromPos: int) -> None:
        L.check(L.lib().skainet_cuda_kv_evict(self.handle, fromPos))

    def clear(self) -> None:
        L.check(L.lib().skainet_cuda_kv_clear(self.handle))

    def decodeStep(self, layer: int, q_ptr: int, out_ptr: int, qHeads: int, fromPos: int, toPos: int, scale: float = 0.0, stream: int = 0) -> None:
        """Attention of one query row per head over positions [fromPos, toPos), read in place from the ring."""
        L.check(L.lib().skainet_cuda_kv_attn_decode_dev(self.handle, layer, q_ptr, out_ptr, qHeads, fromPos, toPos, scale, stream))

    def free(self) -> None:
        if self.handle:
            L.lib().skainet_cuda_kv_free(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
