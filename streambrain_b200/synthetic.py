"""Seeded synthetic stand-ins for the datasets the reference trains on, and the
named workload configurations used by the tests and the benchmark.

The reference's example driver reads MNIST / Fashion-MNIST IDX files and STL-10
binaries (train.py:9-41); none of those files are available offline, so inputs of
the same shapes and value ranges are drawn from a private ``RandomState`` (the
global NumPy stream, which seeds the layers, is left untouched).

Pixels are complementary-coded: pixel ``p`` becomes the unit pair ``(p, 1-p)`` at
positions ``2k, 2k+1``, i.e. one two-minicolumn input hypercolumn per pixel.
Hyper-parameters are the reference's per-dataset defaults (train.py:74-139),
``taupdt`` scaled by ``sqrt(batch/128)`` (train.py:144-145), initial traces
``(1, 1/Mc, 1/Mc)`` for the hidden layer and ``(1/Mc, 1/10, 1/(10 Mc))`` for the
classifier (train.py:163-179).
"""
from __future__ import annotations

import math

import numpy as np

DATA_SEED = 1234


def complementary_code(pixels: np.ndarray) -> np.ndarray:
    out = np.empty((pixels.shape[0], 2 * pixels.shape[1]), dtype=pixels.dtype)
    out[:, 0::2] = pixels
    out[:, 1::2] = 1 - pixels
    return out


def sparse_pixels(rng: np.random.RandomState, n: int, n_pixels: int, sparsity: float, dtype) -> np.ndarray:
    """Each pixel is 0 with probability ``sparsity`` else uniform[0,1)."""
    u = rng.rand(n, n_pixels)
    v = rng.rand(n, n_pixels)
    return np.where(v >= sparsity, u, 0.0).astype(dtype)


def one_hot_labels(rng: np.random.RandomState, n: int, classes: int, dtype) -> np.ndarray:
    lab = rng.randint(0, classes, size=n)
    out = np.zeros((n, classes), dtype=dtype)
    out[np.arange(n), lab] = 1
    return out


def make_inputs(n: int, n_pixels: int, sparsity: float, dtype, seed: int = DATA_SEED,
                classes: int = 10):
    """Return (complementary-coded inputs [n, 2*n_pixels], one-hot labels [n, classes])."""
    rng = np.random.RandomState(seed)
    x = complementary_code(sparse_pixels(rng, n, n_pixels, sparsity, dtype))
    y = one_hot_labels(rng, n, classes, dtype)
    return x, y


_MNIST = dict(taupdt=0.006908854922437549, pmin=0.06195283356566607, khalf=-139.02586632856327,
              taubdt=0.02218100432360414, density=0.1, out_taupdt=0.0007449780036161324)
_STL10 = dict(taupdt=0.0006510421564830368, pmin=0.0070169782620369365, khalf=1666.644815059196,
              taubdt=0.0024793529936481956, density=0.568746541818903, out_taupdt=4.983000352087509e-07)

# name -> workload.  n_pixels*2 = in_features of the hidden layer.
CONFIGS = {
    "mnist_f32": dict(n_pixels=784, sparsity=0.8, H=30, Mc=100, batch=128, dtype="float32", hp=_MNIST),
    "mnist_f64": dict(n_pixels=784, sparsity=0.8, H=30, Mc=100, batch=128, dtype="float64", hp=_MNIST),
    "wide_f32": dict(n_pixels=784, sparsity=0.8, H=100, Mc=300, batch=1024, dtype="float32", hp=_MNIST),
    "stl10_f32": dict(n_pixels=27648, sparsity=0.0, H=30, Mc=100, batch=256, dtype="float32", hp=_STL10),
    # not a reference configuration: the STL-10 shape in float64, to characterise the float64 kernels at a size
    # where launch and pipeline-fill overheads do not dominate
    "stl10_f64": dict(n_pixels=27648, sparsity=0.0, H=30, Mc=100, batch=256, dtype="float64", hp=_STL10),
    "stl10_dp_f32": dict(n_pixels=27648, sparsity=0.0, H=30, Mc=100, batch=8192, dtype="float32", hp=_STL10),
}


def layer_params(name: str, batch: int | None = None) -> dict:
    """Constructor arguments of the hidden and the classifier layer of a workload."""
    c = CONFIGS[name]
    hp = c["hp"]
    batch = batch or c["batch"]
    scale = math.sqrt(batch / 128)
    Mc = c["Mc"]
    hidden = dict(in_features=2 * c["n_pixels"], hypercolumns=c["H"], minicolumns=Mc,
                  taupdt=hp["taupdt"] * scale, khalf=hp["khalf"], pmin=hp["pmin"], taubdt=hp["taubdt"],
                  density=hp["density"], mask_iterations=16, initial_counters=(1, 1 / Mc, 1 / Mc))
    out = dict(in_features=c["H"] * Mc, hypercolumns=1, minicolumns=10, taupdt=hp["out_taupdt"] * scale,
               initial_counters=(1 / Mc, 1 / 10, 1 / Mc / 10))
    return dict(hidden=hidden, out=out, batch=batch, dtype=np.dtype(c["dtype"]),
                n_pixels=c["n_pixels"], sparsity=c["sparsity"])


def steady_state_traces(p, x, seed=7):
    """Traces of a layer that has already seen data, used as the start state of both arms.

    With the constructor's initial traces (Ci = 1, Cij = Cj = 1/Mc) the plasticity score
    log((pj - pij) / ((1 - pi) pj)) is undefined (0/0), which is why the reference never
    updates the mask in its first epoch (_cpu_base_backend.py:297).  The timed steps update
    the mask, so they start where later epochs are: Ci = mean input, Cj = 1/Mc and
    Cij = Ci*Cj (independent units) with 5 % seeded noise."""
    hp = p["hidden"]
    N, M, Mc = hp["in_features"], hp["hypercolumns"] * hp["minicolumns"], hp["minicolumns"]
    rs = np.random.default_rng(seed)
    dt = p["dtype"]
    Ci = np.clip(x.mean(axis=0, dtype=np.float64), 0.02, 0.98).astype(dt)
    Cj = np.full(M, 1.0 / Mc, dtype=dt)
    Cij = (Ci[:, None].astype(np.float32) * Cj[None, :].astype(np.float32))
    Cij *= 1.0 + 0.05 * rs.standard_normal(size=(N, M), dtype=np.float32)
    # keep Cij < Cj (and < Ci): the score takes log((pj - pij) / ...), which a joint trace above its
    # marginal would turn into NaN -- a state the moving averages cannot reach from data
    np.minimum(Cij, 0.98 * np.minimum(Ci[:, None].astype(np.float32), Cj[None, :].astype(np.float32)), out=Cij)
    return Ci, Cj, np.ascontiguousarray(Cij.astype(dt))
