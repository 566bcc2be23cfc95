"""Host-side logic that needs no GPU: the library's batch planner (batch slices per rank, mask
schedule) driving CPU oracle layers through the reference's golden network run, the synthetic data
generator, the dispatcher and the row-block arithmetic of the data-parallel step."""
import importlib
import random

import numpy as np
import pytest

from conftest import TOL, load_golden, rel_inf

import oracle
from streambrain_b200 import parallel, synthetic
from plan_driver import PlanNetwork, plan


class _OraclePlastic(oracle.OracleLayer):
    def __init__(self, k, dtype, *a, **kw):
        super().__init__(k, "plastic", *a, dtype=dtype, **kw)

    def convert(self, dtype):
        raise AssertionError("layers are created in the network dtype")


def _golden_network(port_kernels, tag, dtype, world=(0, 1)):
    g = load_golden("network_%s.npz" % tag)
    n_pix, H, Mc, B = int(g["n_pix"]), int(g["H"]), int(g["Mc"]), int(g["B"])
    n_train = int(g["n_train"])
    seed = int(g["seed"])
    np.random.seed(seed)
    random.seed(seed)
    net = PlanNetwork(np.dtype(dtype))
    l0 = oracle.OracleLayer(port_kernels, "plastic", 2 * n_pix, H, Mc, 0.03, (1, 1 / Mc, 1 / Mc), np.float64,
                            khalf=-40.0, pmin=0.1, taubdt=0.05, density=0.5)
    l1 = oracle.OracleLayer(port_kernels, "dense", H * Mc, 1, 10, 0.02, (1 / Mc, 1 / 10, 1 / Mc / 10), np.float64)
    for l in (l0, l1):  # the reference creates layers in float64 and add_layer converts them
        for name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi"):
            if hasattr(l, name):
                setattr(l, name, getattr(l, name).astype(dtype))
        l.dtype = np.dtype(dtype)
        net.add_layer(l)
    x, lab = g["x"], g["labels"]
    net.fit(x[:n_train], lab[:n_train], B, [(0, 3)])
    net.fit(x[:n_train], lab[:n_train], B, [(1, 2)])
    correct, total = net.evaluate(x[n_train:], lab[n_train:], B)
    return g, net, correct, total


def test_network_driver_reproduces_reference_run_f64(port_kernels):
    g, net, correct, total = _golden_network(port_kernels, "f64", np.float64)
    assert np.array_equal(net.layers[0].wmask, g["l0_wmask"])
    for li, layer in enumerate(net.layers):
        for name in ("Ci", "Cj", "Cij", "bias", "weights"):
            assert rel_inf(getattr(layer, name), g["l%d_%s" % (li, name)]) < 1e-9, (li, name)
    assert int(correct[0]) == int(g["correct"][0]) and int(total[0]) == int(g["total"][0])


def test_network_driver_reproduces_reference_run_f32(port_kernels):
    g, net, correct, total = _golden_network(port_kernels, "f32", np.float32)
    for li, layer in enumerate(net.layers):
        for name in ("Ci", "Cj"):
            assert rel_inf(getattr(layer, name), g["l%d_%s" % (li, name)]) < 1e-3, (li, name)
    assert int(total[0]) == int(g["total"][0])


def test_mask_schedule_needs_enough_batches(port_kernels):
    """Fewer batches than hypercolumns+1 divides by zero in the reference
    (_cpu_base_backend.py:297); the driver keeps that behaviour."""
    net = PlanNetwork(np.float64)
    net.add_layer(oracle.OracleLayer(port_kernels, "plastic", 8, 4, 2, 0.05, (1, 0.5, 0.5), np.float64,
                                     khalf=-10.0, pmin=0.1, taubdt=0.1, density=0.5, rng=np.random.RandomState(0)))
    net.add_layer(oracle.OracleLayer(port_kernels, "dense", 8, 1, 10, 0.05, (0.5, 0.1, 0.05), np.float64,
                                     rng=np.random.RandomState(1)))
    x, lab = synthetic.make_inputs(16, 4, 0.5, np.float64)
    with pytest.raises(ZeroDivisionError):
        net.fit(x, lab, 8, [(0, 2)])
    net.fit(x, lab, 8, [(0, 1)])   # a single epoch never reaches the mask schedule


def test_batch_plan_arithmetic():
    """469 batches of 128 over 60000 samples with 30 hypercolumns: exactly 30 mask updates per later
    epoch, at batches 0, 15, ..., 435, none in the first epoch; the last batch is partial; two ranks
    halve every batch and drop the odd sample."""
    n, bs, H = 60000, 128, 30
    nb = -(-n // bs)
    assert all(plan(n, bs, 1, 0, H, 0, b)[2] == -1 for b in range(nb))
    slots = [(b, plan(n, bs, 1, 0, H, 1, b)[2]) for b in range(nb)]
    assert [b for b, s in slots if s >= 0] == list(range(0, 450, 15))
    assert [s for b, s in slots if s >= 0] == list(range(30))
    assert plan(n, bs, 1, 0, H, 1, nb - 1)[:2] == ((nb - 1) * bs, 96)
    assert plan(35, 10, 2, 1, 2, 0, 3)[:2] == (30 + 2, 2)       # 5 samples left, 2 per rank
    assert plan(35, 10, 2, 0, 2, 0, 1)[:2] == (10, 5)
    with pytest.raises(Exception):
        plan(35, 10, 2, 2, 2, 0, 0)                               # rank outside the world


def test_synthetic_inputs_are_seeded_and_complementary():
    x1, y1 = synthetic.make_inputs(32, 784, 0.8, np.float32)
    x2, y2 = synthetic.make_inputs(32, 784, 0.8, np.float32)
    assert np.array_equal(x1, x2) and np.array_equal(y1, y2)
    assert x1.shape == (32, 1568) and y1.shape == (32, 10)
    assert np.allclose(x1[:, 0::2] + x1[:, 1::2], 1.0)
    assert abs((x1[:, 0::2] == 0).mean() - 0.8) < 0.02
    assert np.array_equal(y1.sum(axis=1), np.ones(32, dtype=np.float32))
    p = synthetic.layer_params("stl10_f32")
    assert p["hidden"]["in_features"] == 55296 and p["hidden"]["hypercolumns"] * p["hidden"]["minicolumns"] == 3000
    assert abs(p["hidden"]["taupdt"] - 0.0006510421564830368 * np.sqrt(2)) < 1e-15


def test_row_blocks_cover_all_rows_on_tile_boundaries():
    for n in (1, 127, 128, 129, 1568, 55296, 3000):
        for blocks in (1, 2, 4, 7, 1000):
            b = parallel.row_block_bounds(n, blocks)
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(lo % 128 == 0 for lo, _ in b)
            assert all(b[k][1] == b[k + 1][0] for k in range(len(b) - 1))
            assert len(b) <= blocks
    lo, hi = parallel.delta_slice(10, 4, 0, 10)
    assert (lo, hi) == (0, 10 + 4 + 40)
    assert parallel.delta_slice(256, 4, 128, 256) == (256 + 4 + 128 * 4, 256 + 4 + 256 * 4)


def test_dispatcher_names(monkeypatch):
    import streambrain_b200
    monkeypatch.setenv("BCPNN_BACKEND", "nonsense")
    mod = importlib.reload(streambrain_b200)
    assert mod.backend() == "nonsense"
    with pytest.raises(ValueError, match="Unable to import backend"):
        mod.Network
    monkeypatch.setenv("BCPNN_BACKEND", "b200")
    mod = importlib.reload(streambrain_b200)
    assert mod.backend() == "b200"
    from streambrain_b200.backend import b200_backend
    assert mod.Network is b200_backend.Network
