"""The view-kernel pack's host logic (skainet_b200/viewpack.py, the tested twin of the Kotlin CudaViewKernelPack): a weight
view is uploaded once per storage OBJECT and found again by identity, the device copy is freed when the storage goes, and
the pack installs every (encoding, block order) once, and only while the provider is available. A recording fake stands in
for the device, so this runs without a GPU; the GPU half is tests/test_gpu_viewpack.py."""
import gc

import numpy as np
import pytest

from skainet_b200 import _lib as L
from skainet_b200.viewpack import (CudaPackedMatmulKernel, CudaViewKernelPack, ENCODINGS, INPUT_MAJOR, KernelDispatch, PackedWeightView,
                                   ROW_MAJOR, key_for)


class FakeDevice:
    def __init__(self):
        self.uploads, self.frees, self.calls = [], [], 0

    def upload(self, packed, encoding, n, k, order):
        h = ("w", len(self.uploads))
        self.uploads.append((h, bytes(packed[:8]), packed.size, encoding, n, k, order))
        return h

    def matmul(self, handle, x, out):
        self.calls += 1
        out[...] = float(handle[1])

    def free(self, handle):
        self.frees.append(handle)


def view(enc, n, k, order=ROW_MAJOR, fill=1, offset=0):
    nbytes = n * (k // L.BLOCK_ELEMS[enc]) * L.BLOCK_BYTES[enc]
    return PackedWeightView(np.full(nbytes + offset, fill, np.uint8), (n, k), enc, order, offset)


def test_weight_is_uploaded_once_per_storage_object_and_freed_with_it():
    dev = FakeDevice()
    kern = CudaPackedMatmulKernel("Q4_K", ROW_MAJOR, dev)
    w1, w2 = view("Q4_K", 8, 512), view("Q4_K", 8, 512)            # equal bytes, two storage objects
    x, out = np.ones((3, 512), np.float32), np.zeros((3, 8), np.float32)
    for _ in range(4):
        kern.run([x, w1], out)
    assert len(dev.uploads) == 1 and dev.calls == 4 and (out == 0.0).all()
    kern.run([x, w2], out)                                          # identity, not content, is the key
    assert len(dev.uploads) == 2 and (out == 1.0).all()
    alias = PackedWeightView(w1.storage, (8, 512), "Q4_K", ROW_MAJOR)      # another view over the SAME storage: no new upload
    kern.run([x, alias], out)
    assert len(dev.uploads) == 2 and (out == 0.0).all()
    assert dev.uploads[0][2:] == (8 * 2 * 144, "Q4_K", 8, 512, ROW_MAJOR)
    del w1, alias
    gc.collect()
    assert dev.frees == [("w", 0)]                                  # the device copy went with its storage
    del w2
    gc.collect()
    assert sorted(dev.frees) == [("w", 0), ("w", 1)]


def test_byte_offset_and_size_of_the_view_are_honoured():
    dev = FakeDevice()
    kern = CudaPackedMatmulKernel("Q6_K", INPUT_MAJOR, dev)
    w = view("Q6_K", 4, 256, INPUT_MAJOR, fill=7, offset=16)
    w.storage[:16] = 0xEE
    kern.run([np.ones((1, 256), np.float32), w], np.zeros((1, 4), np.float32))
    h, head, size, enc, n, k, order = dev.uploads[0]
    assert head == bytes([7] * 8) and size == 4 * 210 and (enc, n, k, order) == ("Q6_K", 4, 256, INPUT_MAJOR)
    short = PackedWeightView(np.zeros(100, np.uint8), (4, 256), "Q6_K", INPUT_MAJOR)
    with pytest.raises(IndexError):
        kern.run([np.ones((1, 256), np.float32), short], np.zeros((1, 4), np.float32))


def test_views_the_kernel_cannot_take_are_refused_by_name():
    dev = FakeDevice()
    kern = CudaPackedMatmulKernel("Q8_0", ROW_MAJOR, dev)
    w = view("Q8_0", 4, 64)
    out = np.zeros((2, 4), np.float32)
    with pytest.raises(ValueError, match="contiguous activation"):
        kern.run([np.ones((2, 128), np.float32)[:, ::2], w], out)
    with pytest.raises(ValueError, match="inner dimensions disagree"):
        kern.run([np.ones((2, 96), np.float32), w], out)
    with pytest.raises(ValueError, match="does not match the key"):
        kern.run([np.ones((2, 64), np.float32), view("Q8_0", 4, 64, INPUT_MAJOR)], out)
    with pytest.raises(ValueError, match="two operands"):
        kern.run([np.ones((2, 64), np.float32)], out)
    with pytest.raises(ValueError, match="output must be"):
        kern.run([np.ones((2, 64), np.float32), w], np.zeros((2, 5), np.float32))
    with pytest.raises(ValueError, match="no GPU view kernel"):
        CudaPackedMatmulKernel("Q4_0", ROW_MAJOR, dev)
    assert dev.uploads == [] and dev.calls == 0                    # nothing reached the device


def test_pack_installs_every_key_once_and_only_when_available():
    dispatch = KernelDispatch()
    CudaViewKernelPack(available=lambda: False, backend=FakeDevice()).install(dispatch)
    assert len(dispatch) == 0                                       # unavailable provider: a no-op, the CPU packs keep serving
    pack = CudaViewKernelPack(available=lambda: True, backend=FakeDevice())
    pack.install(dispatch)
    assert len(dispatch) == 2 * len(ENCODINGS)
    first = dispatch.lookup(key_for("Q5_K", INPUT_MAJOR))
    assert first is not None and first.name == "cuda-sm100-q5_k-im"
    pack.install(dispatch)                                          # idempotent
    assert dispatch.lookup(key_for("Q5_K", INPUT_MAJOR)) is first
    assert dispatch.lookup(key_for("Q4_0", ROW_MAJOR)) is None
