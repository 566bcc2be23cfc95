"""Generate the golden input/output vectors under tests/golden/ from the UNMODIFIED
StreamBrain reference (``BCPNN_BACKEND=cpu``), imported from its checkout.

Needs a reference checkout (environment variable ``SBB_REFERENCE_ROOT``, see
``oracle/build.py``) and the compiled OpenMP module built by ``oracle/build.py``.  The reference cannot
travel to other machines, so the small ``.npz`` files this script writes are
committed and every other consumer reads those.

    python tests/golden/make_golden.py

Cases (both float32 and float64):
  kernels_<dtype>.npz   one call of every kernel wrapper of the cpu backend
                        (kernels_openmp.py + kernels_numpy.py) on seeded inputs.
  layer_<dtype>.npz     a StructuralPlasticityLayer trained for 14 steps through
                        compute_activation/train_step (mask updates from step 3),
                        state recorded after every step; a DenseLayer trained on
                        the hidden activations, with train_finalize.
  network_<dtype>.npz   Network.fit (hidden layer 3 epochs incl. the mask schedule,
                        classifier 2 epochs) + Network.evaluate on a tiny dataset.
"""
from __future__ import annotations

import os
import random
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REPO, "oracle"))

import build as oracle_build  # noqa: E402
from streambrain_b200 import synthetic  # noqa: E402


def import_reference():
    root = oracle_build.reference_root()
    if root is None:
        raise SystemExit("no reference checkout found")
    mod = oracle_build.build_reference()
    sys.path.insert(0, os.path.dirname(mod))
    sys.path.insert(0, root)
    os.environ["BCPNN_BACKEND"] = "cpu"
    import BCPNN
    from BCPNN.backend._kernels import kernels_numpy, kernels_openmp
    return BCPNN, kernels_openmp, kernels_numpy


def kernel_vectors(k_omp, k_np, dtype, seed):
    rs = np.random.RandomState(seed)
    out = {}
    B, N, H, Mc = 9, 37, 3, 7
    M = H * Mc
    # update_state + softmax
    x = rs.rand(B, N).astype(dtype)
    w = (0.3 * rs.randn(N, M)).astype(dtype)
    b = rs.randn(M).astype(dtype)
    s = k_omp.update_state(np.zeros((B, M), dtype=dtype), w, b, x)
    out.update(us_x=x, us_w=w, us_b=b, us_out=s.copy())
    out["sm_out"] = k_np.softmax_minicolumns(s.copy(), H, Mc).astype(dtype)
    # fused update_weights
    taupdt = 0.05
    Ci = rs.rand(N).astype(dtype)
    Cj = rs.rand(M).astype(dtype)
    Cij = rs.rand(N, M).astype(dtype)
    Ci[3] = 0.001  # below cthr -> zero row
    Cj[5] = 0.0    # below cthr -> zero column
    y = k_np.softmax_minicolumns(rs.randn(B, M), H, Mc).astype(dtype)
    out.update(uw_Ci=Ci.copy(), uw_Cj=Cj.copy(), uw_Cij=Cij.copy(), uw_x=x, uw_y=y, uw_taupdt=taupdt)
    Ci2, Cj2, Cij2, W2 = k_omp.update_weights(Ci.copy(), Cj.copy(), Cij.copy(), x, y, taupdt,
                                              np.full((N, M), 7.0, dtype=dtype), taupdt / 2)
    out.update(uw_Ci_out=Ci2, uw_Cj_out=Cj2, uw_Cij_out=Cij2, uw_W_out=W2)
    # un-fused numpy pair
    c1, c2, c3 = k_np.update_counters(Ci.copy(), Cj.copy(), Cij.copy(), x, y, taupdt)
    out.update(uc_Ci_out=c1.astype(dtype), uc_Cj_out=c2.astype(dtype), uc_Cij_out=c3.astype(dtype))
    out["rw_W_out"] = k_np.update_weights(np.zeros((N, M), dtype=dtype), c1, c2, c3, taupdt / 2).astype(dtype)
    # bias kernels
    out["ub_out"] = k_omp.update_bias(np.zeros(M, dtype=dtype), Cj2.copy(), taupdt / 2)
    kbi = (10 * rs.randn(M)).astype(dtype)
    khalf, pmin, taubdt = -139.0, 0.3, 0.02
    bb, kk = k_omp.update_bias_regularized(np.zeros(M, dtype=dtype), kbi.copy(), Cj2.copy(), taupdt / 2,
                                           khalf, pmin, taubdt)
    out.update(ubr_kbi=kbi, ubr_khalf=khalf, ubr_pmin=pmin, ubr_taubdt=taubdt, ubr_bias_out=bb, ubr_kbi_out=kk)
    # update_mask with finite logs (recipe of _kernels/test_openmp.py:185-233), 1 and 16 iterations
    n, hc, mc = 53, 4, 6
    m = hc * mc
    wmask = (rs.rand(n, hc) < 0.3).astype(np.uint8)
    mw = (0.1 * rs.randn(n, m)).astype(dtype)
    mCi = rs.rand(n).astype(dtype)
    mCj = rs.rand(m).astype(dtype)
    mCij = np.minimum(np.minimum(0.9 * mCi[:, None], 0.9 * mCj[None, :]), rs.rand(n, m)).astype(dtype)
    out.update(um_wmask=wmask, um_w=mw, um_Ci=mCi, um_Cj=mCj, um_Cij=mCij, um_cthr=0.01)
    for it in (1, 16):
        for h in range(hc):
            out["um_out_it%d_h%d" % (it, h)] = k_omp.update_mask(wmask.copy(), mw, mCi, mCj, mCij, 0.01,
                                                                 hc, mc, h, it)
    out["am_out"] = k_omp.apply_mask(mw.copy(), wmask, hc, mc)
    return out


def layer_trajectory(BCPNN, dtype, seed):
    out = {}
    n_pix, H, Mc, B, steps = 24, 4, 6, 16, 14
    N, M = 2 * n_pix, H * Mc
    x_all, lab_all = synthetic.make_inputs(B * steps, n_pix, 0.5, dtype, seed=seed)
    np.random.seed(seed)
    hp = dict(taupdt=0.02, khalf=-50.0, pmin=0.1, taubdt=0.05, density=0.4)
    layer = BCPNN.StructuralPlasticityLayer(N, H, Mc, hp["taupdt"], hp["khalf"], hp["pmin"], hp["taubdt"],
                                            hp["density"], 16, (1, 1 / Mc, 1 / Mc), dtype=dtype)
    dense = BCPNN.DenseLayer(M, 1, 10, 0.01, (1 / Mc, 1 / 10, 1 / Mc / 10), dtype=dtype)
    out.update(n_pix=n_pix, H=H, Mc=Mc, B=B, steps=steps, seed=seed, x=x_all, labels=lab_all,
               **{"hp_" + k: v for k, v in hp.items()}, dense_taupdt=0.01)
    for name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask"):
        out["init_" + name] = getattr(layer, name).copy()
    for name in ("weights", "bias", "Ci", "Cj", "Cij"):
        out["dinit_" + name] = getattr(dense, name).copy()
    hs = []
    for s in range(steps):
        x = x_all[s * B:(s + 1) * B]
        lab = lab_all[s * B:(s + 1) * B]
        act = layer.compute_activation(x)
        h = (s * 3) % H if s >= 3 else None
        hs.append(-1 if h is None else h)
        dense_pred = dense.compute_activation(act)
        dense.train_step(act, lab)
        layer.train_step(x, act, h)
        out["act_%d" % s] = act.copy()
        out["dact_%d" % s] = dense_pred.copy()
        for name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask"):
            out["s%d_%s" % (s, name)] = getattr(layer, name).copy()
        for name in ("weights", "Ci", "Cj", "Cij"):
            out["d%d_%s" % (s, name)] = getattr(dense, name).copy()
    dense.train_finalize()
    out["dfinal_bias"] = dense.bias.copy()
    out["hs"] = np.array(hs)
    return out


def network_run(BCPNN, dtype, seed):
    n_pix, H, Mc, B = 16, 3, 5, 8
    n_train, n_test = 8 * 9 + 3, 21  # partial last batch on purpose
    x, lab = synthetic.make_inputs(n_train + n_test, n_pix, 0.5, dtype, seed=seed)
    np.random.seed(seed)
    random.seed(seed)
    net = BCPNN.Network(dtype)
    net.add_layer(BCPNN.StructuralPlasticityLayer(2 * n_pix, H, Mc, 0.03, -40.0, 0.1, 0.05, 0.5, 16,
                                                  (1, 1 / Mc, 1 / Mc)))
    net.add_layer(BCPNN.DenseLayer(H * Mc, 1, 10, 0.02, (1 / Mc, 1 / 10, 1 / Mc / 10)))
    net.fit(x[:n_train], lab[:n_train], B, [(0, 3)])
    net.fit(x[:n_train], lab[:n_train], B, [(1, 2)])
    correct, total = net.evaluate(x[n_train:], lab[n_train:], B)
    out = dict(n_pix=n_pix, H=H, Mc=Mc, B=B, n_train=n_train, n_test=n_test, seed=seed, x=x, labels=lab,
               correct=correct, total=total)
    for li, layer in enumerate(net._layers):
        for name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask"):
            if hasattr(layer, name):
                out["l%d_%s" % (li, name)] = getattr(layer, name).copy()
    act = x[n_train:]
    for layer in net._layers:
        act = layer.compute_activation(act)
    out["test_pred"] = np.argmax(act, axis=1)
    return out


def main():
    BCPNN, k_omp, k_np = import_reference()
    for dtype, tag in ((np.float32, "f32"), (np.float64, "f64")):
        np.savez_compressed(os.path.join(HERE, "kernels_%s.npz" % tag), **kernel_vectors(k_omp, k_np, dtype, 11))
        np.savez_compressed(os.path.join(HERE, "layer_%s.npz" % tag), **layer_trajectory(BCPNN, dtype, 5))
        np.savez_compressed(os.path.join(HERE, "network_%s.npz" % tag), **network_run(BCPNN, dtype, 7))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
