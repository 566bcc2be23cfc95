"""The allocation-free mask update (sbb_update_mask_noalloc) against the ordinary
entry point (sbb_update_mask).

Some hosts of the library own all device memory themselves or cannot tolerate the
device-wide stall of cudaMalloc inside their loop; for them the library keeps the
two per-row work arrays of the mask update in a fixed array of its own.  The test
calls that entry point through the C ABI on caller-owned device buffers, twice in a
row (the second call is smaller and uses another hypercolumn, so it runs over the
first call's left-overs in the shared work area), and requires the resulting masks
to be identical to those of the allocating entry point.  It also checks that a
layer larger than the built-in work area is refused with a clear error.

This file sorts last on purpose: it is collected after every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(rs, n, hc, mc, dtype):
    m = hc * mc
    wmask = (rs.rand(n, hc) < 0.3).astype(np.uint8)
    w = (0.1 * rs.randn(n, m)).astype(dtype)
    Ci = rs.rand(n).astype(dtype)
    Cj = rs.rand(m).astype(dtype)
    Cij = np.minimum(np.minimum(0.9 * Ci[:, None], 0.9 * Cj[None, :]), rs.rand(n, m).astype(dtype)).astype(dtype)
    return wmask, w, Ci, Cj, Cij


def _noalloc(lib, torch, dtype, wmask, w, Ci, Cj, Cij, cthr, hc, mc, h, iterations):
    dev = [torch.from_numpy(a).cuda() for a in (wmask, w, Ci, Cj, Cij)]
    n, m = w.shape
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.sbb_update_mask_noalloc(0 if dtype == np.float32 else 1, dev[0].data_ptr(), dev[1].data_ptr(),
                                     dev[2].data_ptr(), dev[3].data_ptr(), dev[4].data_ptr(), cthr, n, m, hc, mc, h,
                                     iterations, stream)
    assert rc == 0, lib.sbb_noalloc_last_error()
    torch.cuda.synchronize()
    return dev[0].cpu().numpy()


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_noalloc_mask_update_matches_allocating_entry_point(dtype, port_kernels):
    import torch
    from streambrain_b200 import kernels_b200 as k
    from streambrain_b200._lib import lib
    rs = np.random.RandomState(17)
    # two calls in a row: a large case, then a smaller one on another hypercolumn
    for n, hc, mc, h, iterations in ((6000, 5, 40, 3, 16), (700, 4, 25, 1, 16)):
        wmask, w, Ci, Cj, Cij = _case(rs, n, hc, mc, dtype)
        want = k.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, hc, mc, h, iterations)
        got = _noalloc(lib, torch, dtype, wmask.copy(), w, Ci, Cj, Cij, 0.01, hc, mc, h, iterations)
        assert np.array_equal(got, want), (n, h)
        if dtype == np.float64:   # and directly against the CPU statement of the algorithm
            cpu = port_kernels.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, hc, mc, h, iterations)
            assert np.array_equal(got, cpu), (n, h)
        assert not np.array_equal(got, wmask)   # the update did move connections


def test_noalloc_refuses_oversized_layers_without_launching():
    import torch
    from streambrain_b200._lib import lib
    before = int(lib.sbb_kernel_launches())
    one = torch.zeros(8, dtype=torch.float32, device="cuda")
    mask = torch.zeros(8, dtype=torch.uint8, device="cuda")
    n = 131072 + 1
    rc = lib.sbb_update_mask_noalloc(0, mask.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                     one.data_ptr(), 0.01, n, 4, 2, 2, 0, 1, None)
    assert rc == 4
    assert b"131072" in lib.sbb_noalloc_last_error()
    assert int(lib.sbb_kernel_launches()) == before
    assert lib.sbb_update_mask_noalloc(0, None, None, None, None, None, 0.01, 8, 4, 2, 2, 0, 1, None) == 1
