"""CPU restatement of the reference's dense KV-cache store and of attention over a ring window — TEST
INFRASTRUCTURE ONLY (the checker of skainet_cuda_kv_*; nothing the product ships imports it).

Follows skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/DefaultKvCacheStore.kt
(:76-103 appendToken, :105-131 readKeys / readValues / evict, :170-177 slotOf / windowStart, :235-263 readRange)
and skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/memory/WindowedAttention.kt:32-80
(decodeStep: online softmax over the window's positions, oldest first). With f16=True the stored values are
rounded through binary16, which is what the device store holds.
"""
from __future__ import annotations

import numpy as np


class CpuKvStore:
    def __init__(self, numLayers: int, numHeads: int, headDim: int, maxSeqLen: int, slidingWindow: bool = False, f16: bool = False):
        self.numLayers, self.numHeads, self.headDim, self.maxSeqLen = numLayers, numHeads, headDim, maxSeqLen
        self.slidingWindow, self.f16 = slidingWindow, f16
        self.currentSeqLen = 0
        self.keys = np.zeros((numLayers, numHeads, maxSeqLen, headDim), np.float32)
        self.values = np.zeros_like(self.keys)

    def _slot(self, position: int) -> int:
        return position % self.maxSeqLen if self.slidingWindow else position

    @property
    def windowStart(self) -> int:
        return max(self.currentSeqLen - self.maxSeqLen, 0) if self.slidingWindow else 0

    def _store(self, x: np.ndarray) -> np.ndarray:
        x = np.asarray(x, np.float32)
        return x.astype(np.float16).astype(np.float32) if self.f16 else x

    def appendToken(self, layer: int, key: np.ndarray, value: np.ndarray) -> None:
        if not 0 <= layer < self.numLayers:
            raise ValueError(f"Layer index {layer} out of range [0, {self.numLayers})")
        if not (self.slidingWindow or self.currentSeqLen < self.maxSeqLen):
            raise RuntimeError(f"KV cache is full: currentSeqLen={self.currentSeqLen}, maxSeqLen={self.maxSeqLen}")
        n = self.numHeads * self.headDim
        if np.size(key) != n or np.size(value) != n:
            raise ValueError("Key/Value size mismatch")
        pos = self._slot(self.currentSeqLen)
        self.keys[layer, :, pos, :] = self._store(key).reshape(self.numHeads, self.headDim)
        self.values[layer, :, pos, :] = self._store(value).reshape(self.numHeads, self.headDim)
        if layer == self.numLayers - 1:
            self.currentSeqLen += 1

    def _read(self, data: np.ndarray, layer: int, startPos: int, endPos: int) -> np.ndarray:
        if not (self.windowStart <= startPos <= endPos):
            raise ValueError(f"Invalid range: startPos={startPos}, endPos={endPos}, oldest held position={self.windowStart}")
        if endPos > self.currentSeqLen:
            raise ValueError(f"endPos={endPos} exceeds currentSeqLen={self.currentSeqLen}")
        slots = [self._slot(p) for p in range(startPos, endPos)]
        return data[layer][:, slots, :].copy()

    def readKeys(self, layer: int, startPos: int = 0, endPos: int | None = None) -> np.ndarray:
        return self._read(self.keys, layer, startPos, self.currentSeqLen if endPos is None else endPos)

    def readValues(self, layer: int, startPos: int = 0, endPos: int | None = None) -> np.ndarray:
        return self._read(self.values, layer, startPos, self.currentSeqLen if endPos is None else endPos)

    def evict(self, fromPos: int) -> None:
        if not 0 <= fromPos <= self.currentSeqLen:
            raise ValueError(f"evict fromPos={fromPos} out of range [0, {self.currentSeqLen}]")
        self.currentSeqLen = fromPos
        if fromPos < self.maxSeqLen:
            self.keys[:, :, fromPos:, :] = 0.0
            self.values[:, :, fromPos:, :] = 0.0

    def clear(self) -> None:
        self.currentSeqLen = 0
        self.keys[:] = 0.0
        self.values[:] = 0.0


def windowed_decode_step(query: np.ndarray, keys: np.ndarray, values: np.ndarray, scale: float = 0.0) -> np.ndarray:
    """query [heads, headDim]; keys / values [heads, positions, headDim] in position order (the runs of a window
    concatenated oldest first). fp32 online softmax exactly in the order decodeStep takes."""
    heads, npos, hd = keys.shape
    s = np.float32(scale) if scale != 0.0 else np.float32(1.0) / np.sqrt(np.float32(hd))
    out = np.zeros((heads, hd), np.float32)
    q = np.asarray(query, np.float32).reshape(heads, hd)
    for h in range(heads):
        running_max = -np.inf
        denom = np.float32(0.0)
        acc = np.zeros(hd, np.float32)
        for p in range(npos):
            score = np.float32(0.0)
            for d in range(hd):
                score = np.float32(score + q[h, d] * keys[h, p, d])
            score = np.float32(score * s)
            new_max = max(running_max, score)
            corr = np.float32(0.0) if running_max == -np.inf else np.float32(np.exp(np.float32(running_max - new_max)))
            w = np.float32(np.exp(np.float32(score - new_max)))
            denom = np.float32(denom * corr + w)
            acc = (acc * corr + w * values[h, p]).astype(np.float32)
            running_max = new_max
        out[h] = acc / denom
    return out
