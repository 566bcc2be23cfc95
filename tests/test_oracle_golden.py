"""Pins the CPU oracle (the plain-C restatement) against golden vectors that were
produced by the unmodified StreamBrain `cpu` backend (tests/golden/make_golden.py).
Runs without a GPU."""
import numpy as np
import pytest

from conftest import TOL, load_golden, rel_inf, weight_err

import oracle

DTYPES = [("f32", np.float32), ("f64", np.float64)]


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_kernels_match_reference(port_kernels, tag, dtype):
    g = load_golden("kernels_%s.npz" % tag)
    k = port_kernels
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
        assert rel_inf(got, g[name]) < tol
    W2 = k.recompute_weights(np.zeros((N, M), dtype=dtype), g["uc_Ci_out"], g["uc_Cj_out"], g["uc_Cij_out"], t / 2)
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
            assert np.array_equal(got, g["um_out_it%d_h%d" % (it, h)]), (it, h)
    assert np.array_equal(k.apply_mask(g["um_w"].copy(), g["um_wmask"], hc, mc), g["am_out"])


def _layers_from_golden(g, kernels, dtype):
    H, Mc, n_pix = int(g["H"]), int(g["Mc"]), int(g["n_pix"])
    layer = oracle.OracleLayer(kernels, "plastic", 2 * n_pix, H, Mc, float(g["hp_taupdt"]), (1, 1 / Mc, 1 / Mc),
                               dtype, khalf=float(g["hp_khalf"]), pmin=float(g["hp_pmin"]),
                               taubdt=float(g["hp_taubdt"]), density=float(g["hp_density"]),
                               rng=np.random.RandomState(0))
    dense = oracle.OracleLayer(kernels, "dense", H * Mc, 1, 10, float(g["dense_taupdt"]),
                               (1 / Mc, 1 / 10, 1 / Mc / 10), dtype, rng=np.random.RandomState(0))
    for name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask"):
        setattr(layer, name, g["init_" + name].copy())
    for name in ("weights", "bias", "Ci", "Cj", "Cij"):
        setattr(dense, name, g["dinit_" + name].copy())
    return layer, dense


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_layer_steps_teacher_forced(port_kernels, tag, dtype):
    """Each step starts from the reference's recorded state, so errors cannot compound."""
    g = load_golden("layer_%s.npz" % tag)
    tol = TOL[np.dtype(dtype)]
    layer, dense = _layers_from_golden(g, port_kernels, dtype)
    B, steps = int(g["B"]), int(g["steps"])
    for s in range(steps):
        x = g["x"][s * B:(s + 1) * B]
        lab = g["labels"][s * B:(s + 1) * B]
        act = layer.compute_activation(x)
        assert rel_inf(act, g["act_%d" % s]) < tol, s
        assert rel_inf(dense.compute_activation(g["act_%d" % s]), g["dact_%d" % s]) < tol, s
        h = int(g["hs"][s])
        dense.train_step(g["act_%d" % s], lab)
        layer.train_step(x, g["act_%d" % s], None if h < 0 else h)
        for name in ("Ci", "Cj", "Cij", "kbi", "bias"):
            assert rel_inf(getattr(layer, name), g["s%d_%s" % (s, name)]) < tol, (s, name)
        assert weight_err(layer.weights, g["s%d_weights" % s]) < 10 * tol, s
        assert np.array_equal(layer.wmask, g["s%d_wmask" % s]), s
        for name in ("Ci", "Cj", "Cij"):
            assert rel_inf(getattr(dense, name), g["d%d_%s" % (s, name)]) < tol, (s, name)
        assert weight_err(dense.weights, g["d%d_weights" % s]) < 10 * tol, s
        for name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask"):
            setattr(layer, name, g["s%d_%s" % (s, name)].copy())
        for name in ("weights", "Ci", "Cj", "Cij"):
            setattr(dense, name, g["d%d_%s" % (s, name)].copy())
    dense.train_finalize()
    assert rel_inf(dense.bias, g["dfinal_bias"]) < tol


def test_layer_free_run_f64(port_kernels):
    """Float64 free run: 14 steps without resetting to the reference state; masks must be identical."""
    g = load_golden("layer_f64.npz")
    layer, _ = _layers_from_golden(g, port_kernels, np.float64)
    B, steps = int(g["B"]), int(g["steps"])
    for s in range(steps):
        x = g["x"][s * B:(s + 1) * B]
        act = layer.compute_activation(x)
        h = int(g["hs"][s])
        layer.train_step(x, act, None if h < 0 else h)
        assert np.array_equal(layer.wmask, g["s%d_wmask" % s]), s
    assert rel_inf(layer.Cij, g["s%d_Cij" % (steps - 1)]) < 1e-10
    assert rel_inf(layer.weights, g["s%d_weights" % (steps - 1)]) < 1e-9


def test_reference_module_agrees_with_port(port_kernels):
    """When the compiled reference module is present, run both on a fresh random case."""
    try:
        ref = oracle.RefKernels()
    except Exception as e:  # pragma: no cover - depends on the machine
        pytest.skip("compiled reference not available: %s" % e)
    rs = np.random.RandomState(3)
    for dtype in (np.float32, np.float64):
        B, N, M = 33, 130, 77
        x = rs.rand(B, N).astype(dtype)
        y = rs.rand(B, M).astype(dtype)
        st = [rs.rand(N).astype(dtype), rs.rand(M).astype(dtype), rs.rand(N, M).astype(dtype)]
        a = ref.update_weights(*[v.copy() for v in st], x, y, 0.01, np.zeros((N, M), dtype=dtype), 0.005)
        b = port_kernels.update_weights(*[v.copy() for v in st], x, y, 0.01, np.zeros((N, M), dtype=dtype), 0.005)
        for u, v in zip(a, b):
            assert rel_inf(v, u) < TOL[np.dtype(dtype)]
