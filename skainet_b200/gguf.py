"""GGUF tensors straight to the device: the host-side mirror of the reference's streaming reader
(skainet-io/skainet-io-gguf/src/commonMain/kotlin/sk/ainet/io/gguf/StreamingGGUFReader.kt:60-139: `fields`, `tensors`,
`loadTensorData`) for the part of the format the packed decode path needs. The header, the metadata and the tensor
infos are parsed; a tensor's bytes are read from the file where they lie (memory-mapped) and handed to
skainet_cuda_weight_upload in the file's own row-major block order, which is the order the kernels take. Written from the
published GGUF layout (magic, version 2/3, little endian, counted strings, typed metadata values, tensor infos with
dimensions innermost first and offsets relative to the aligned data section)."""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Any, Dict, List

import numpy as np

from ._lib import BLOCK_BYTES, BLOCK_ELEMS, ENC_NAME

GGUF_MAGIC = 0x46554747          # "GGUF"
GGML_F32, GGML_F16 = 0, 1
# ggml type ids of the packed encodings are the library's SKAINET_ENC_* values (8 Q8_0, 12 Q4_K, 13 Q5_K, 14 Q6_K)
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


@dataclass
class StreamingTensorInfo:
    name: str
    shape: tuple          # outermost first: (rows = out, cols = in) for a matrix
    ggml_type: int
    offset: int           # relative to the data section
    absoluteDataOffset: int
    nBytes: int

    @property
    def encoding(self) -> str | None:
        return ENC_NAME.get(self.ggml_type)


class StreamingGGUFReader:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.fields: Dict[str, Any] = {}
        self.tensors: List[StreamingTensorInfo] = []
        self._parse()

    # ---- parsing -----------------------------------------------------------------------------------------------
    def _u(self, fmt: str, pos: int):
        return struct.unpack_from(fmt, self._mm, pos)[0], pos + struct.calcsize(fmt)

    def _string(self, pos: int):
        n, pos = self._u("<Q", pos)
        return bytes(self._mm[pos:pos + n]).decode("utf-8", "replace"), pos + n

    def _value(self, vtype: int, pos: int):
        if vtype in _SCALAR:
            return self._u(_SCALAR[vtype], pos)
        if vtype == _STRING:
            return self._string(pos)
        if vtype == _ARRAY:
            et, pos = self._u("<I", pos)
            n, pos = self._u("<Q", pos)
            out = []
            for _ in range(n):
                v, pos = self._value(et, pos)
                out.append(v)
            return out, pos
        raise ValueError(f"GGUF: unknown metadata value type {vtype}")

    def _parse(self) -> None:
        magic, pos = self._u("<I", 0)
        if magic != GGUF_MAGIC:
            raise ValueError("not a GGUF file")
        self.version, pos = self._u("<I", pos)
        if self.version not in (2, 3):
            raise ValueError(f"GGUF version {self.version} not supported")
        n_tensors, pos = self._u("<Q", pos)
        n_kv, pos = self._u("<Q", pos)
        for _ in range(n_kv):
            key, pos = self._string(pos)
            vt, pos = self._u("<I", pos)
            self.fields[key], pos = self._value(vt, pos)
        raw = []
        for _ in range(n_tensors):
            name, pos = self._string(pos)
            nd, pos = self._u("<I", pos)
            dims = []
            for _ in range(nd):
                d, pos = self._u("<Q", pos)
                dims.append(d)
            t, pos = self._u("<I", pos)
            off, pos = self._u("<Q", pos)
            raw.append((name, tuple(reversed(dims)), t, off))
        align = int(self.fields.get("general.alignment", 32))
        data_start = (pos + align - 1) // align * align
        for name, shape, t, off in raw:
            self.tensors.append(StreamingTensorInfo(name, shape, t, off, data_start + off, self._nbytes(shape, t)))

    @staticmethod
    def _nbytes(shape: tuple, t: int) -> int:
        n = int(np.prod(shape)) if shape else 1
        if t == GGML_F32:
            return 4 * n
        if t == GGML_F16:
            return 2 * n
        enc = ENC_NAME.get(t)
        if enc is None:
            raise ValueError(f"GGUF: tensor type {t} has no decoder here")
        if shape[-1] % BLOCK_ELEMS[enc]:
            raise ValueError(f"GGUF: innermost dimension {shape[-1]} is not a whole number of {enc} blocks")
        return n // BLOCK_ELEMS[enc] * BLOCK_BYTES[enc]

    # ---- loading -----------------------------------------------------------------------------------------------------
    def tensor(self, name: str) -> StreamingTensorInfo:
        for t in self.tensors:
            if t.name == name:
                return t
        raise ValueError(f"Tensor not found: {name}")

    def loadTensorData(self, tensor: StreamingTensorInfo) -> np.ndarray:
        """The tensor's raw bytes, a view of the mapped file (nothing is copied until it is used)."""
        return np.frombuffer(self._mm, dtype=np.uint8, count=tensor.nBytes, offset=tensor.absoluteDataOffset)

    def loadTensor(self, name: str) -> np.ndarray:
        return self.loadTensorData(self.tensor(name))

    def loadWeightToDevice(self, name: str):
        """A packed matrix [rows = out, cols = in] of the file as a resident weight: the mapped bytes go to the device as
        they are (GGUF stores blocks row-major, which is what the kernels take)."""
        from .device import Weight
        t = self.tensor(name)
        if t.encoding is None or len(t.shape) != 2:
            raise ValueError(f"{name}: not a packed matrix (type {t.ggml_type}, shape {t.shape})")
        return Weight.upload(self.loadTensorData(t), t.encoding, t.shape[0], t.shape[1])

    def loadFloats(self, name: str) -> np.ndarray:
        t = self.tensor(name)
        if t.ggml_type != GGML_F32:
            raise ValueError(f"{name}: not an F32 tensor")
        return self.loadTensorData(t).view(np.float32).reshape(t.shape)

    def close(self) -> None:
        self._mm.close()
        self._f.close()
