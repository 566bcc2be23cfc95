"""The reference's own kernel test contract, run against this repository's kernel modules.

StreamBrain tests a kernel module by ``run_tests(k1, kernels_numpy)`` of
``BCPNN/backend/_kernels/test_openmp.py:256-309``: random shapes, float64 data, every kernel compared
with the NumPy kernels at 1e-3.  ``oracle/build.py`` stages that script (unmodified, git-ignored) where a
reference checkout is present; here it is run (a) against the reference's own compiled OpenMP module, on
the CPU, to show the staged contract is the live one, and (b) on the GPU against ``kernels_b200`` and
against the pybind11 module ``_bcpnn_kernels_b200_internal`` behind the reference's wrapper file.
"""
import importlib
import os
import random
import sys

import numpy as np
import pytest

from conftest import REPO

sys.path.insert(0, os.path.join(REPO, "oracle"))
import build as oracle_build  # noqa: E402


def _contract():
    d = oracle_build.stage_reference_contract()
    mod = oracle_build.ref_module_path()
    if d is None or not os.path.exists(mod):
        pytest.skip("the reference's test script is not staged (no reference checkout was present at build time)")
    for p in (d, os.path.dirname(mod)):
        if p not in sys.path:
            sys.path.insert(0, p)
    return importlib.import_module("test_openmp"), importlib.import_module("kernels_numpy")


def _run(contract, k1, k2):
    random.seed(12)
    np.random.seed(12)
    # run_tests reads the module-level names _k1 / _k2 that its __main__ block sets (test_openmp.py:312-314)
    contract._k1, contract._k2 = k1, k2
    diff, args = contract.run_tests(k1, k2)
    assert diff is None, ("the reference's run_tests reported a difference of %r" % diff)


def test_staged_contract_passes_on_the_reference_itself():
    contract, kernels_numpy = _contract()
    _run(contract, importlib.import_module("kernels_openmp"), kernels_numpy)


@pytest.mark.gpu
def test_reference_contract_on_the_b200_kernel_module(contraction_path):
    contract, kernels_numpy = _contract()
    from streambrain_b200 import kernels_b200
    _run(contract, kernels_b200, kernels_numpy)


@pytest.mark.gpu
def test_reference_wrapper_file_over_the_pybind_module(contraction_path):
    """kernels_openmp.py of the reference, unmodified, with `_i` bound to the pybind11 module of this
    repository: what a maintainer gets by changing one import line."""
    contract, kernels_numpy = _contract()
    from streambrain_b200 import build as sbb_build
    path = sbb_build.pybind_module_path()
    if not os.path.exists(path):
        pytest.skip("the pybind11 module was not built")
    sys.path.insert(0, os.path.dirname(path))
    shim = importlib.import_module("_bcpnn_kernels_b200_internal")
    wrapper = importlib.import_module("kernels_openmp")
    saved = wrapper._i
    try:
        wrapper._i = shim
        # the reference's apply_mask test passes an int8 mask (test_openmp.py:243), which this module
        # accepts for a mask that is only read
        _run(contract, wrapper, kernels_numpy)
    finally:
        wrapper._i = saved


@pytest.mark.gpu
def test_pybind_module_matches_the_ctypes_binding_and_rejects_silent_copies(contraction_path):
    from streambrain_b200 import build as sbb_build, kernels_b200 as k
    path = sbb_build.pybind_module_path()
    if not os.path.exists(path):
        pytest.skip("the pybind11 module was not built")
    sys.path.insert(0, os.path.dirname(path))
    m = importlib.import_module("_bcpnn_kernels_b200_internal")
    assert m.initialize() >= 1
    rs = np.random.RandomState(0)
    for dtype, sfx in ((np.float32, "_float32"), (np.float64, "_float64")):
        B, N, H, Mc = 9, 20, 3, 4
        M = H * Mc
        x, w, b = rs.rand(B, N).astype(dtype), rs.randn(N, M).astype(dtype), rs.randn(M).astype(dtype)
        out = np.zeros((B, M), dtype=dtype)
        getattr(m, "update_state" + sfx)(out, x, w, b)
        assert np.array_equal(out, k.update_state(np.zeros((B, M), dtype=dtype), w, b, x))
        out2 = np.zeros((B, M), dtype=dtype)
        getattr(m, "update_state_cuda_order" + sfx)(out2, w, b, x)
        assert np.array_equal(out, out2)
        sm = out.copy()
        getattr(m, "softmax_minicolumns" + sfx)(sm, H, Mc)
        assert np.array_equal(sm, k.softmax_minicolumns(out.copy(), H, Mc))
        st = [rs.rand(N).astype(dtype), rs.rand(M).astype(dtype), rs.rand(N, M).astype(dtype)]
        y = rs.rand(B, M).astype(dtype)
        a = [v.copy() for v in st] + [np.zeros((N, M), dtype=dtype)]
        c = getattr(m, "update_weights" + sfx)(1.0, a[0], a[1], a[2], x, y, 0.1, a[3], 0.05)
        want = k.update_weights(*[v.copy() for v in st], x, y, 0.1, np.zeros((N, M), dtype=dtype), 0.05)
        assert all(np.array_equal(p, q) for p, q in zip(a, want)) and abs(c - 1.0) < 1e-6
        w2 = np.zeros((N, M), dtype=dtype)
        getattr(m, "update_weights" + sfx)(w2, a[0], a[1], a[2], 0.05)          # the gpu module's un-fused form
        assert np.array_equal(w2, k.update_weights(np.zeros((N, M), dtype=dtype), a[0], a[1], a[2], 0.05))
        mask = (rs.rand(N, H) < 0.4).astype(np.uint8)
        got = mask.copy()
        getattr(m, "update_mask" + sfx)(got, w, a[0], a[1], np.minimum(a[2], 0.5 * np.minimum.outer(a[0], a[1])), 0.01,
                                        H, Mc, 1, 4)
        want = k.update_mask(mask.copy(), w, a[0], a[1], np.minimum(a[2], 0.5 * np.minimum.outer(a[0], a[1])), 0.01,
                             H, Mc, 1, 4)
        assert np.array_equal(got, want)
        wm = w.copy()
        getattr(m, "apply_mask" + sfx)(wm, mask.astype(np.int8), H, Mc)
        assert np.array_equal(wm, k.apply_mask(w.copy(), mask, H, Mc))
    with pytest.raises(TypeError):     # float64 state with the float32 function: no silent conversion
        m.update_state_float32(np.zeros((2, 2)), np.zeros((2, 2), np.float32), np.zeros((2, 2), np.float32),
                               np.zeros(2, np.float32))
    with pytest.raises(TypeError):     # a mask that is written must be uint8
        m.update_mask_float64(np.zeros((2, 1), np.int8), np.zeros((2, 2)), np.zeros(2), np.zeros(2), np.zeros((2, 2)),
                              0.1, 1, 2, 0, 1)
