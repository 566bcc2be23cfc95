"""Kernel-level parity on the GPU, through the C ABI (streambrain_b200.kernels_b200):
against the golden vectors of the reference cpu backend, and -- in the style of the
reference's own fuzz tests (_kernels/test_openmp.py, test_cuda.py) but for float32
as well as float64 and with odd sizes -- against the CPU oracle on seeded inputs."""
import numpy as np
import pytest

from conftest import TOL, load_golden, mask_mismatch_is_a_tie, rel_inf, weight_err

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("contraction_path")]

DTYPES = [("f32", np.float32), ("f64", np.float64)]


@pytest.fixture(scope="module")
def k():
    from streambrain_b200 import kernels_b200
    return kernels_b200


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_kernels_match_reference_golden(k, tag, dtype):
    g = load_golden("kernels_%s.npz" % tag)
    tol = TOL[np.dtype(dtype)]
    B, N = g["us_x"].shape
    M = g["us_w"].shape[1]
    H, Mc = 3, 7
    s = k.update_state(np.zeros((B, M), dtype=dtype), g["us_w"], g["us_b"], g["us_x"])
    assert rel_inf(s, g["us_out"]) < tol
    assert rel_inf(k.softmax_minicolumns(g["us_out"].copy(), H, Mc), g["sm_out"]) < tol

    t = float(g["uw_taupdt"])
    Ci, Cj, Cij, W = k.update_weights(g["uw_Ci"].copy(), g["uw_Cj"].copy(), g["uw_Cij"].copy(), g["uw_x"],
                                      g["uw_y"], t, np.full((N, M), 7.0, dtype=dtype), t / 2)
    assert rel_inf(Ci, g["uw_Ci_out"]) < tol
    assert rel_inf(Cj, g["uw_Cj_out"]) < tol
    assert rel_inf(Cij, g["uw_Cij_out"]) < tol
    assert weight_err(W, g["uw_W_out"]) < 10 * tol
    assert np.array_equal(W == 0, g["uw_W_out"] == 0)

    c = k.update_counters(g["uw_Ci"].copy(), g["uw_Cj"].copy(), g["uw_Cij"].copy(), g["uw_x"], g["uw_y"], t)
    for got, name in zip(c, ("uc_Ci_out", "uc_Cj_out", "uc_Cij_out")):
        assert rel_inf(got, g[name]) < tol, name
    W2 = k.update_weights(np.zeros((N, M), dtype=dtype), g["uc_Ci_out"], g["uc_Cj_out"], g["uc_Cij_out"], t / 2)
    assert weight_err(W2, g["rw_W_out"]) < 10 * tol

    assert rel_inf(k.update_bias(np.zeros(M, dtype=dtype), g["uw_Cj_out"].copy(), t / 2), g["ub_out"]) < tol
    b, kb = k.update_bias_regularized(np.zeros(M, dtype=dtype), g["ubr_kbi"].copy(), g["uw_Cj_out"].copy(), t / 2,
                                      float(g["ubr_khalf"]), float(g["ubr_pmin"]), float(g["ubr_taubdt"]))
    assert rel_inf(b, g["ubr_bias_out"]) < tol
    assert rel_inf(kb, g["ubr_kbi_out"]) < tol

    hc, mc = 4, 6
    for it in (1, 16):
        for h in range(hc):
            got = k.update_mask(g["um_wmask"].copy(), g["um_w"], g["um_Ci"], g["um_Cj"], g["um_Cij"],
                                float(g["um_cthr"]), hc, mc, h, it)
            if dtype == np.float64:
                assert np.array_equal(got, g["um_out_it%d_h%d" % (it, h)]), (it, h)
            else:  # float32: a different swap only where the reference's own margin is below the score noise
                want = g["um_out_it%d_h%d" % (it, h)]
                ref_state = {"Ci": g["um_Ci"], "Cj": g["um_Cj"], "Cij": g["um_Cij"]}
                assert mask_mismatch_is_a_tie(got, want, h, g["um_wmask"], ref_state, float(g["um_cthr"]), mc,
                                              1e-5), (it, h)
    assert np.array_equal(k.apply_mask(g["um_w"].copy(), g["um_wmask"], hc, mc), g["am_out"])


SHAPES = [(1, 1, 1, 1), (3, 5, 1, 2), (7, 129, 3, 43), (33, 257, 5, 13), (100, 1000, 30, 10), (128, 64, 2, 300),
          (65, 130, 1, 1024), (17, 520, 7, 19),
          # rows that are 16-byte multiples: eligible for the tensor-core kernels
          (5, 4, 1, 4), (77, 388, 3, 44), (300, 260, 2, 130), (16, 2048, 1, 260), (130, 132, 4, 65)]


@pytest.mark.parametrize("tag,dtype", DTYPES)
@pytest.mark.parametrize("B,N,H,Mc", SHAPES)
def test_forward_and_softmax_vs_oracle(k, port_kernels, tag, dtype, B, N, H, Mc):
    rs = np.random.RandomState(B * 7 + N)
    M = H * Mc
    x = rs.randn(B, N).astype(dtype)
    w = rs.randn(N, M).astype(dtype)
    b = rs.randn(M).astype(dtype)
    got = k.update_state(np.zeros((B, M), dtype=dtype), w, b, x)
    want = port_kernels.update_state(np.zeros((B, M), dtype=dtype), w, b, x)
    assert rel_inf(got, want) < TOL[np.dtype(dtype)]
    a = (3 * rs.randn(B, M)).astype(dtype)
    got = k.softmax_minicolumns(a.copy(), H, Mc)
    want = port_kernels.softmax_minicolumns(a.copy(), H, Mc)
    assert rel_inf(got, want) < TOL[np.dtype(dtype)]
    assert np.allclose(got.reshape(B, H, Mc).sum(axis=2), 1.0, atol=1e-5)
    z = k.add_bias(a.copy(), b)
    assert np.array_equal(z, a + b)


@pytest.mark.parametrize("tag,dtype", DTYPES)
@pytest.mark.parametrize("B,N,H,Mc", SHAPES)
def test_trace_update_vs_oracle(k, port_kernels, tag, dtype, B, N, H, Mc):
    rs = np.random.RandomState(B * 11 + N)
    M = H * Mc
    tol = TOL[np.dtype(dtype)]
    st = [rs.rand(N).astype(dtype), rs.rand(M).astype(dtype), rs.rand(N, M).astype(dtype)]
    st[0][rs.rand(N) < 0.1] = 0   # 10% exact zeros, as the reference's C++ fuzz harness seeds them
    st[1][rs.rand(M) < 0.1] = 0
    st[2][rs.rand(N, M) < 0.1] = 0
    x = rs.rand(B, N).astype(dtype)
    y = rs.rand(B, M).astype(dtype)
    taupdt = 0.01 + 0.5 * rs.rand()
    got = k.update_weights(*[v.copy() for v in st], x, y, taupdt, np.zeros((N, M), dtype=dtype), taupdt / 2)
    want = port_kernels.update_weights(*[v.copy() for v in st], x, y, taupdt, np.zeros((N, M), dtype=dtype),
                                       taupdt / 2)
    for a, b_, name in zip(got, want, ("Ci", "Cj", "Cij", "W")):
        assert (weight_err(a, b_) < 10 * tol) if name == "W" else (rel_inf(a, b_) < tol), name
    assert np.array_equal(got[3] == 0, want[3] == 0)
    got = k.update_counters(*[v.copy() for v in st], x, y, taupdt)
    want = port_kernels.update_counters(*[v.copy() for v in st], x, y, taupdt)
    for a, b_ in zip(got, want):
        assert rel_inf(a, b_) < tol
    w1 = k.update_weights(np.zeros((N, M), dtype=dtype), *want, taupdt / 2)
    w2 = port_kernels.recompute_weights(np.zeros((N, M), dtype=dtype), *want, taupdt / 2)
    assert weight_err(w1, w2) < 10 * tol


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_bias_kernels_vs_oracle(k, port_kernels, tag, dtype):
    rs = np.random.RandomState(5)
    tol = TOL[np.dtype(dtype)]
    for M in (1, 31, 1000, 3000):
        Cj = rs.rand(M).astype(dtype)
        Cj[::7] = 0
        cthr = 0.05
        assert rel_inf(k.update_bias(np.zeros(M, dtype=dtype), Cj, cthr),
                       port_kernels.update_bias(np.zeros(M, dtype=dtype), Cj, cthr)) < tol
        kbi = (10 * rs.randn(M)).astype(dtype)
        khalf, pmin, taubdt = -100 - 900 * rs.rand(), rs.rand(), rs.rand()
        b1, k1 = k.update_bias_regularized(np.zeros(M, dtype=dtype), kbi.copy(), Cj, cthr, khalf, pmin, taubdt)
        b2, k2 = port_kernels.update_bias_regularized(np.zeros(M, dtype=dtype), kbi.copy(), Cj, cthr, khalf, pmin,
                                                      taubdt)
        assert rel_inf(b1, b2) < tol and rel_inf(k1, k2) < tol


def _mask_case(rs, n, hc, mc, dtype, density=0.3):
    m = hc * mc
    wmask = (rs.rand(n, hc) < density).astype(np.uint8)
    w = (0.1 * rs.randn(n, m)).astype(dtype)
    Ci = rs.rand(n).astype(dtype)
    Cj = rs.rand(m).astype(dtype)
    Cij = np.minimum(np.minimum(0.9 * Ci[:, None], 0.9 * Cj[None, :]), rs.rand(n, m).astype(dtype)).astype(dtype)
    return wmask, w, Ci, Cj, Cij


@pytest.mark.parametrize("n,hc,mc", [(1, 1, 2), (53, 4, 6), (128, 2, 64), (700, 3, 100), (2500, 30, 10),
                                     # 1024 rows and more take the candidate-list search instead of the full scan
                                     (1024, 2, 8), (4096, 2, 8), (5000, 3, 20), (30011, 2, 10)])
def test_update_mask_f64_identical_to_oracle(k, port_kernels, n, hc, mc):
    rs = np.random.RandomState(n)
    wmask, w, Ci, Cj, Cij = _mask_case(rs, n, hc, mc, np.float64)
    for it in (1, 16, 32, 40):
        for h in sorted({0, hc - 1, hc // 2}):
            got = k.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, hc, mc, h, it)
            want = port_kernels.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, hc, mc, h, it)
            assert np.array_equal(got, want), (it, h)
    assert np.array_equal(k.apply_mask(w.copy(), wmask, hc, mc), port_kernels.apply_mask(w.copy(), wmask, hc, mc))


def test_update_mask_edge_cases(k, port_kernels):
    rs = np.random.RandomState(2)
    wmask, w, Ci, Cj, Cij = _mask_case(rs, 40, 2, 5, np.float64)
    for fill in (0, 1):   # nothing silent / nothing active: no swap possible
        m = np.full_like(wmask, fill)
        assert np.array_equal(k.update_mask(m.copy(), w, Ci, Cj, Cij, 0.01, 2, 5, 1, 16), m)
    # exact ties: identical rows must resolve to the last index, as the sequential scan does
    Ci[:] = 0.5
    Cij[:] = 0.1
    w[:] = 0.2
    got = k.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, 2, 5, 0, 3)
    want = port_kernels.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, 2, 5, 0, 3)
    assert np.array_equal(got, want)
    # zero iterations leaves the mask alone
    assert np.array_equal(k.update_mask(wmask.copy(), w, Ci, Cj, Cij, 0.01, 2, 5, 0, 0), wmask)


@pytest.mark.parametrize("n", [1500, 6000])
@pytest.mark.parametrize("iterations", [3, 16, 32])
def test_update_mask_with_nan_scores_at_the_head_of_a_class(k, port_kernels, n, iterations):
    """Always-on inputs (Ci == 1 and Cij == Cj) give NaN scores.  The reference's scan picks a NaN
    row exactly when it is the lowest-index row of its class, which can repeat swap after swap
    (the row heads the other class next) -- the candidate-list search must follow it move by move.
    Several low rows of both classes are made NaN, among them row 0 and the first silent row."""
    rs = np.random.RandomState(7 * n + iterations)
    wmask, w, Ci, Cj, Cij = _mask_case(rs, n, 3, 6, np.float64, density=0.5)
    with np.errstate(all="ignore"):
        for h in range(3):
            Ci2, Cij2 = Ci.copy(), Cij.copy()
            first_silent = int(np.flatnonzero(wmask[:, h] == 0)[0])
            first_active = int(np.flatnonzero(wmask[:, h] == 1)[0])
            hot = sorted({0, 1, 2, 5, 9, first_silent, first_active, n // 2, n - 1})
            Ci2[hot] = 1.0
            Cij2[hot] = Cj[None, :]
            got = k.update_mask(wmask.copy(), w, Ci2, Cj, Cij2, 0.01, 3, 6, h, iterations)
            want = port_kernels.update_mask(wmask.copy(), w, Ci2, Cj, Cij2, 0.01, 3, 6, h, iterations)
            assert np.array_equal(got, want), (h, np.flatnonzero((got != want).any(axis=1))[:10])


@pytest.mark.parametrize("n", [300, 6000])
def test_update_mask_with_nan_and_inf_scores(k, port_kernels, n):
    """Rows whose Ci is exactly 1 (an input that is always on) divide by zero in the score:
    +-inf and NaN scores must be ranked exactly as the reference's front-to-back scan ranks
    them, in the full scan (small n) and in the candidate-list search."""
    rs = np.random.RandomState(n)
    wmask, w, Ci, Cj, Cij = _mask_case(rs, n, 3, 6, np.float64, density=0.4)
    for variant in range(3):
        Ci2, Cij2 = Ci.copy(), Cij.copy()
        hot = rs.choice(n, size=7, replace=False)
        Ci2[hot] = 1.0
        if variant == 1:
            Cij2[hot[:3]] = Cj[None, :]          # pj - pij == 0 -> 0 * log(0/0): NaN
        if variant == 2:
            Ci2[0] = 1.0                          # the very first candidate of its class
            Cij2[0] = Cj
        with np.errstate(all="ignore"):
            for h in range(3):
                got = k.update_mask(wmask.copy(), w, Ci2, Cj, Cij2, 0.01, 3, 6, h, 16)
                want = port_kernels.update_mask(wmask.copy(), w, Ci2, Cj, Cij2, 0.01, 3, 6, h, 16)
                assert np.array_equal(got, want), (variant, h)


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(k):
    """The tensor-core kernels bound every wait on a barrier by a time limit.  With the limit set to about a
    millisecond and one barrier arrival withheld (a test hook of the library) the waiting warp must give up in
    order: the launch returns, the status word names the wait, the entry point reports SBB_ERR_TIMEOUT, and after
    clearing the word the same call works again on the same device."""
    import ctypes
    from streambrain_b200 import _lib
    from streambrain_b200._lib import lib
    if lib.sbb_get_contraction_path() != 1 or not lib.sbb_tensor_path_available():
        pytest.skip("the bounded waits belong to the tensor-core kernels")
    rs = np.random.RandomState(3)
    x, w, b = rs.rand(64, 256).astype(np.float32), rs.randn(256, 128).astype(np.float32), rs.randn(128).astype(np.float32)
    want = k.update_state(np.zeros((64, 128), dtype=np.float32), w, b, x)
    before = lib.sbb_get_wait_limit_cycles()
    try:
        assert lib.sbb_set_wait_limit_cycles(2_000_000) == 0
        assert lib.sbb_debug_lose_arrival(1) == 0
        k.update_state(np.zeros((64, 128), dtype=np.float32), w, b, x)      # result undefined, must return
        status = ctypes.c_int(0)
        assert lib.sbb_device_wait_status(ctypes.byref(status)) == _lib.ERR_TIMEOUT
        assert status.value == 3                                             # the MMA warp's wait for a converted stage
        assert lib.sbb_stream_sync(None) == _lib.ERR_TIMEOUT                 # sticky until cleared
    finally:
        lib.sbb_debug_lose_arrival(0)
        lib.sbb_set_wait_limit_cycles(before)
        assert lib.sbb_device_clear_wait_status() == 0
    got = k.update_state(np.zeros((64, 128), dtype=np.float32), w, b, x)
    assert np.array_equal(got, want)
    status = ctypes.c_int(7)
    assert lib.sbb_device_wait_status(ctypes.byref(status)) == 0 and status.value == 0


def test_one_cta_form_of_the_tensor_kernels(port_kernels, tmp_path):
    """The tensor-core contractions run as CTA pairs by default; SBB_TC_PAIR=0 (read once per process, hence the
    child process) keeps one CTA per tile.  Both forms of the forward product, of the single-chain and of the
    multi-chain trace update must agree with the oracle."""
    import os
    import subprocess
    import sys
    from conftest import REPO
    script = r'''
import sys
import numpy as np
sys.path.insert(0, %r)
from streambrain_b200 import kernels_b200 as k
from streambrain_b200._lib import check, lib
check(lib.sbb_set_contraction_path(1))
out = {}
for tag, (B, N, H, Mc) in {"single": (256, 388, 3, 44), "multi": (600, 260, 2, 130)}.items():
    rs = np.random.RandomState(B + N)
    M = H * Mc
    x, y = rs.rand(B, N).astype(np.float32), rs.rand(B, M).astype(np.float32)
    st = [rs.rand(N).astype(np.float32), rs.rand(M).astype(np.float32), rs.rand(N, M).astype(np.float32)]
    w = rs.randn(N, M).astype(np.float32)
    b = rs.randn(M).astype(np.float32)
    out[tag + "_fwd"] = k.update_state(np.zeros((B, M), dtype=np.float32), w, b, x)
    got = k.update_weights(*[v.copy() for v in st], x, y, 0.05, np.zeros((N, M), dtype=np.float32), 0.025)
    for name, v in zip(("Ci", "Cj", "Cij", "W"), got):
        out[tag + "_" + name] = v
np.savez(sys.argv[1], **out)
''' % REPO
    results = {}
    for pair in ("0", "1"):
        path = str(tmp_path / ("pair%s.npz" % pair))
        env = dict(os.environ, SBB_TC_PAIR=pair)
        subprocess.run([sys.executable, "-c", script, path], check=True, env=env, timeout=300)
        results[pair] = np.load(path)
    tol = TOL[np.dtype(np.float32)]
    for tag, (B, N, H, Mc) in {"single": (256, 388, 3, 44), "multi": (600, 260, 2, 130)}.items():
        rs = np.random.RandomState(B + N)
        M = H * Mc
        x, y = rs.rand(B, N).astype(np.float32), rs.rand(B, M).astype(np.float32)
        st = [rs.rand(N).astype(np.float32), rs.rand(M).astype(np.float32), rs.rand(N, M).astype(np.float32)]
        w = rs.randn(N, M).astype(np.float32)
        b = rs.randn(M).astype(np.float32)
        fwd = port_kernels.update_state(np.zeros((B, M), dtype=np.float32), w, b, x)
        want = port_kernels.update_weights(*[v.copy() for v in st], x, y, 0.05, np.zeros((N, M), dtype=np.float32), 0.025)
        for pair in ("0", "1"):
            r = results[pair]
            assert rel_inf(r[tag + "_fwd"], fwd) < tol, (tag, pair)
            for name, v in zip(("Ci", "Cj", "Cij"), want):
                assert rel_inf(r[tag + "_" + name], v) < tol, (tag, pair, name)
            assert weight_err(r[tag + "_W"], want[3]) < 10 * tol, (tag, pair)
