"""The view-kernel pack against the device: x . W^T over packed weight views in both block orders through the installed
kernels, compared with the reference's C kernels; the weight crosses PCIe once per storage object."""
import gc

import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu


def test_installed_view_kernels_match_the_reference_and_keep_weights_resident(gpu, oracle):
    from skainet_b200.viewpack import CudaViewKernelPack, DeviceBackend, INPUT_MAJOR, KernelDispatch, PackedWeightView, ROW_MAJOR, key_for

    class Counting(DeviceBackend):
        uploads = frees = 0

        def upload(self, *a):
            Counting.uploads += 1
            return super().upload(*a)

        def free(self, handle):
            Counting.frees += 1
            super().free(handle)

    dispatch = KernelDispatch()
    CudaViewKernelPack(backend=Counting()).install(dispatch)
    assert len(dispatch) == 8
    use_ref = oracle.ref() is not None
    rng = np.random.default_rng(11)
    n, k, m = 96, 1024, 3
    x = rng.standard_normal((m, k)).astype(np.float32)
    for enc in ("Q4_K", "Q8_0", "Q6_K", "Q5_K"):
        if enc in ("Q4_K", "Q8_0"):
            wf = (0.03 * rng.standard_normal((n, k))).astype(np.float32)
            packed = oracle.quantize_q4k(wf) if enc == "Q4_K" else oracle.quantize_q8_0(wf)
        else:
            packed = oracle.random_kquant_blocks(enc, n, k, seed=n + k)
        ref = oracle.matmul(enc, x, packed, k, n, "rm", use_ref=use_ref).reshape(m, n)
        for order in (ROW_MAJOR, INPUT_MAJOR):
            before = Counting.uploads
            stored = packed.copy() if order == ROW_MAJOR else oracle.to_feed_order(packed, enc, n, k)
            view = PackedWeightView(stored, (n, k), enc, order)
            kern = dispatch.lookup(key_for(enc, order))
            out = np.zeros((m, n), np.float32)
            kern.run([x, view], out)
            rel_err_ok(out, ref, 1e-3 if enc in ("Q4_K", "Q8_0") else 1e-4)
            first = out.copy()
            kern.run([x, view], out)                     # the second call finds the device copy by the storage's identity
            np.testing.assert_array_equal(out, first)
            assert Counting.uploads == before + 1
            del view, stored
    gc.collect()
    assert Counting.frees == Counting.uploads == 8       # every device copy went with its storage
