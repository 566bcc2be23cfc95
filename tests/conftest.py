import os
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (REPO, os.path.join(REPO, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(REPO, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name)) as z:
        return {k: z[k] for k in z.files}


def rel_inf(a, b):
    """Norm-wise relative error  max|a-b| / max|b|  (0 when both are all-zero)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.abs(b).max() if b.size else 0.0
    num = np.abs(a - b).max() if b.size else 0.0
    return 0.0 if num == 0.0 else num / max(den, 1e-300)


def weight_err(w, ref):
    """Error of a weight matrix relative to max(1, max|ref|).  Weights are logarithms of trace
    ratios and enter the forward sum next to biases of order one, so an absolute scale of one
    is the meaningful floor when every weight happens to be tiny (independent units)."""
    w = np.asarray(w, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return np.abs(w - ref).max() / max(1.0, np.abs(ref).max())


def mask_mismatch_is_a_tie(got, want, h, before, ref_state, cthr, Mc, noise):
    """A float32 mask may differ from the reference's only where the reference's own
    choice was decided by less than the float32 score noise.  Scores are recomputed
    in float64 from the reference's post-update traces."""
    if np.array_equal(got, want):
        return True
    if not np.array_equal(np.delete(got, h, axis=1), np.delete(want, h, axis=1)):
        return False
    if got[:, h].sum() != want[:, h].sum():
        return False
    cols = slice(h * Mc, (h + 1) * Mc)
    Ci, Cj = ref_state["Ci"].astype(np.float64), ref_state["Cj"].astype(np.float64)
    pij, pi, pj = ref_state["Cij"][:, cols].astype(np.float64), Ci[:, None], Cj[None, cols]
    with np.errstate(all="ignore"):
        w = np.log(np.maximum(pij, cthr ** 4) / (pi * pj))
        term = pij * w + (pj - pij) * np.log((pj - pij) / ((1 - pi) * pj))
    nom = np.where((pi >= cthr) & (pj >= cthr), term, 0.0).sum(axis=1)
    score = nom / (1.0 + before.sum(axis=1))
    diff = np.flatnonzero(got[:, h] != want[:, h])
    spread = score[diff].max() - score[diff].min()
    return spread <= noise * max(1.0, np.abs(score).max())


# Parity tolerances of the path (relative, norm-wise): activations and traces within
# 1e-5 in float32 and 1e-12 in float64 of the reference `cpu` backend.
TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}


@pytest.fixture(scope="session")
def port_kernels():
    import oracle
    return oracle.PortKernels()


@pytest.fixture(params=["general", "tensor"])
def contraction_path(request):
    """Runs a GPU test once per contraction path: the general-shape FFMA kernels and the
    tcgen05 tensor-core kernels (which fall back to the former for float64 and for shapes
    whose rows are not 16-byte multiples).  After the test the status word of the bounded
    device-side waits must be clear."""
    import ctypes
    from streambrain_b200._lib import lib
    if request.param == "tensor" and not lib.sbb_tensor_path_available():
        pytest.skip("tensor-core path not available on this device")
    before = lib.sbb_get_contraction_path()
    assert lib.sbb_set_contraction_path(1 if request.param == "tensor" else 0) == 0
    yield request.param
    status = ctypes.c_int(0)
    rc = lib.sbb_device_wait_status(ctypes.byref(status))
    lib.sbb_set_contraction_path(before)
    assert rc == 0 and status.value == 0, "a bounded device-side wait gave up (code %d)" % status.value
