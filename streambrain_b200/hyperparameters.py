"""Per-dataset hyper-parameters of the reference's training driver and the network they build.

The values are StreamBrain's ``train.py:74-139``; both trace time constants are scaled by
``sqrt(batch_size / 128)`` (train.py:144-145); the hidden layer has 3000 units split into the
dataset's number of hypercolumns (train.py:147-149); initial traces are ``(1, 1/Mc, 1/Mc)`` for the
hidden layer and ``(1/Mc, 1/10, 1/(10 Mc))`` for the classifier (train.py:151-179).
"""
from __future__ import annotations

import math

import numpy as np

DATASETS = {
    "mnist": dict(n_inputs=28 * 28, n_hypercolumns=15, l1_taupdt=0.006908854922437549, l1_pmin=0.06195283356566607,
                  l1_khalf=-139.02586632856327, l1_taubdt=0.02218100432360414, l1_density=0.1, l1_mask_iterations=16,
                  l2_taupdt=0.0007449780036161324, l1_epochs=30, l2_epochs=60),
    "fashion_mnist": dict(n_inputs=28 * 28, n_hypercolumns=30, l1_taupdt=0.0014712266428529468,
                          l1_pmin=0.10328182984859212, l1_khalf=-160.06386313883948,
                          l1_taubdt=0.0008418555122620076, l1_density=0.1, l1_mask_iterations=16,
                          l2_taupdt=0.00202951854188782, l1_epochs=30, l2_epochs=60),
    "stl-10": dict(n_inputs=3 * 96 * 96, n_hypercolumns=15, l1_taupdt=0.0006510421564830368,
                   l1_pmin=0.0070169782620369365, l1_khalf=1666.644815059196, l1_taubdt=0.0024793529936481956,
                   l1_density=0.568746541818903, l1_mask_iterations=584, l2_taupdt=4.983000352087509e-07,
                   l1_epochs=100, l2_epochs=20),
}

N_HIDDEN = 3000
N_OUTPUTS = 10


def for_dataset(dataset: str, batch_size: int, n_inputs: int | None = None, n_hypercolumns: int | None = None) -> dict:
    """The driver's settings for ``dataset`` at ``batch_size`` (time constants already scaled)."""
    if dataset not in DATASETS:
        raise ValueError("Unknown dataset")
    hp = dict(DATASETS[dataset])
    scale = math.sqrt(batch_size / 128)
    hp["l1_taupdt"] *= scale
    hp["l2_taupdt"] *= scale
    if n_inputs is not None:
        hp["n_inputs"] = n_inputs
    if n_hypercolumns is not None:
        hp["n_hypercolumns"] = n_hypercolumns
    hp["n_minicolumns"] = N_HIDDEN // hp["n_hypercolumns"]
    hp["n_hidden"] = hp["n_hypercolumns"] * hp["n_minicolumns"]
    hp["batch_size"] = batch_size
    return hp


def build_network(backend, hp: dict, precision=np.float32):
    """The two-layer network of train.py:151-179 on ``backend`` (a module exporting ``Network``,
    ``StructuralPlasticityLayer`` and ``DenseLayer``, e.g. :mod:`streambrain_b200`)."""
    mc = hp["n_minicolumns"]
    net = backend.Network(precision)
    net.add_layer(backend.StructuralPlasticityLayer(hp["n_inputs"], hp["n_hypercolumns"], mc, hp["l1_taupdt"],
                                                    hp["l1_khalf"], hp["l1_pmin"], hp["l1_taubdt"], hp["l1_density"],
                                                    hp["l1_mask_iterations"], (1, 1 / mc, 1 * 1 / mc)))
    net.add_layer(backend.DenseLayer(hp["n_hidden"], 1, N_OUTPUTS, hp["l2_taupdt"], (1 / mc, 1 / 10, 1 / mc * 1 / 10)))
    return net
