"""Host-side handle of the device KV-cache store (include/skainet_cuda.h, section 3): the mirror of the reference's
KvCacheStore interface — appendToken / readKeys / readValues / evict / clear / currentSeqLen / windowStart
(skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/KvCacheStore.kt:125-157,
DefaultKvCacheStore.kt:30-36,170-177) — with the cache resident in HBM as binary16 and attention reading it in place."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


class DeviceKvCacheStore:
    def __init__(self, numLayers: int, numHeads: int, headDim: int, maxSeqLen: int, slidingWindow: bool = False):
        h = C.c_int64()
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
