"""Test infrastructure: the fit / evaluate loops over arbitrary Python layer objects, scheduled by the
library's own planner (``sbb_network_batch_plan``).

The shipped ``Network`` runs its loops inside the C library on device-resident layers.  Its host logic
-- which samples a rank takes of which batch, when which hypercolumn's mask is updated, the order of
the random draws -- is the planner plus a few lines of driver; this class repeats those few lines over
CPU layers so that the planner can be checked against the reference's golden run without a GPU."""
import ctypes

import numpy as np

from streambrain_b200 import _lib
from streambrain_b200._lib import lib


def plan(samples, batch_size, world, rank, hypercolumns, epoch, batch):
    first, count, slot = ctypes.c_long(0), ctypes.c_long(0), ctypes.c_long(0)
    rc = lib.sbb_network_batch_plan(samples, batch_size, world, rank, hypercolumns, epoch, batch, ctypes.byref(first),
                                    ctypes.byref(count), ctypes.byref(slot))
    if rc == _lib.ERR_UNSUPPORTED:
        raise ZeroDivisionError(lib.sbb_last_error().decode())
    _lib.check(rc)
    return first.value, count.value, slot.value


class PlanNetwork:
    def __init__(self, dtype, rank=0, world=1):
        self.dtype, self.rank, self.world = np.dtype(dtype), rank, world
        self.layers = []

    def add_layer(self, layer):
        self.layers.append(layer)

    def fit(self, data, labels, batch_size, schedule):
        data, labels = data.astype(self.dtype), labels.astype(self.dtype)
        n = data.shape[0]
        nb = -(-n // batch_size)
        for li, epochs in schedule:
            target = self.layers[li]
            for epoch in range(epochs):
                order = np.random.permutation(range(n))
                hc_order = np.random.permutation(range(target.hypercolumns))
                for b in range(nb):
                    first, count, slot = plan(n, batch_size, self.world, self.rank, target.hypercolumns, epoch, b)
                    rows = order[first:first + count]
                    acts = [data[rows]]
                    for layer in self.layers[:li + 1]:
                        acts.append(layer.compute_activation(acts[-1]))
                    if li + 1 == len(self.layers):
                        target.train_step(acts[-2], labels[rows])
                    else:
                        target.train_step(acts[-2], acts[-1], None if slot < 0 else hc_order[slot])
                target.train_finalize()

    def evaluate(self, data, labels, batch_size):
        data, labels = data.astype(self.dtype), labels.astype(self.dtype)
        n = data.shape[0]
        correct = total = 0
        for b in range(-(-n // batch_size)):
            first, count, _ = plan(n, batch_size, self.world, self.rank, 1, 0, b)
            if count > 0:
                act = data[first:first + count]
                for layer in self.layers:
                    act = layer.compute_activation(act)
                correct += int((np.argmax(act, axis=1) == np.argmax(labels[first:first + count], axis=1)).sum())
            total += count
        return np.array([correct]), np.array([total])
