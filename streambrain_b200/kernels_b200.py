"""Kernel-wrapper module of the B200 backend.

Exports the union of the function names of StreamBrain's kernel-wrapper modules,
with the same argument order, in-place mutation and return values
(BCPNN/backend/_kernels/kernels_openmp.py:6-99 and kernels_cuda.py:8-135), so a
test written against those modules (``run_tests(k1, kernels_numpy)`` of
``_kernels/test_openmp.py:256-309`` / ``test_cuda.py:238-301``) runs against this
one unchanged.  Every call stages the numpy arrays through the current CUDA
device via the C ABI; the device-resident layer path is in
``streambrain_b200.backend.b200_backend``.

Arrays must be C-contiguous and of the dtype of the call: nothing is copied or
converted silently, a mismatch raises ``TypeError``; an unsupported dtype raises
``Exception("Invalid dtype")`` as the reference wrappers do.
"""
from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import check, dtype_code, host_ptr, lib


def update_state(state, weights, bias, inputs):
    dt = state.dtype
    code = dtype_code(dt)
    B, N = inputs.shape
    M = weights.shape[1]
    if weights.shape[0] != N or state.shape != (B, M) or bias.shape != (M,):
        raise ValueError("update_state: shape mismatch")
    check(lib.sbb_update_state(code, host_ptr(state, dt, "state"), host_ptr(inputs, dt, "inputs"),
                               host_ptr(weights, dt, "weights"), host_ptr(bias, dt, "bias"), B, N, M))
    return state


def add_bias(a, x):
    dt = a.dtype
    rows, M = a.shape
    if x.shape != (M,):
        raise ValueError("add_bias: shape mismatch")
    check(lib.sbb_add_bias(dtype_code(dt), host_ptr(a, dt, "a"), host_ptr(x, dt, "x"), rows, M))
    return a


def softmax_minicolumns(a, hypercolumns, minicolumns):
    dt = a.dtype
    code = dtype_code(dt)
    M = hypercolumns * minicolumns
    if a.size % M:
        raise ValueError("softmax_minicolumns: size is not a multiple of hypercolumns*minicolumns")
    check(lib.sbb_softmax_minicolumns(code, host_ptr(a, dt, "a"), a.size // M, hypercolumns, minicolumns))
    return a


def update_counters(Ci, Cj, Cij, a_i, a_o, taupdt):
    dt = Ci.dtype
    code = dtype_code(dt)
    B, N = a_i.shape
    M = a_o.shape[1]
    if Ci.shape != (N,) or Cj.shape != (M,) or Cij.shape != (N, M) or a_o.shape[0] != B:
        raise ValueError("update_counters: shape mismatch")
    check(lib.sbb_update_counters(code, host_ptr(Ci, dt, "Ci"), host_ptr(Cj, dt, "Cj"), host_ptr(Cij, dt, "Cij"),
                                  host_ptr(a_i, dt, "a_i"), host_ptr(a_o, dt, "a_o"), float(taupdt), B, N, M))
    return Ci, Cj, Cij


def update_weights(*args):
    """Two reference signatures share this name:

    * fused, OpenMP module: ``update_weights(Ci, Cj, Cij, a_i, a_o, taupdt, weights, cthr)``
      -> ``(Ci, Cj, Cij, weights)`` (kernels_openmp.py:16-25);
    * un-fused, CUDA/NumPy modules: ``update_weights(weights, Ci, Cj, Cij, cthr)``
      -> ``weights`` (kernels_cuda.py:51-59).
    """
    if len(args) == 8:
        Ci, Cj, Cij, a_i, a_o, taupdt, weights, cthr = args
        dt = Ci.dtype
        code = dtype_code(dt)
        B, N = a_i.shape
        M = a_o.shape[1]
        if Ci.shape != (N,) or Cj.shape != (M,) or Cij.shape != (N, M) or weights.shape != (N, M) \
                or a_o.shape[0] != B:
            raise ValueError("update_weights: shape mismatch")
        check(lib.sbb_update_weights(code, host_ptr(Ci, dt, "Ci"), host_ptr(Cj, dt, "Cj"), host_ptr(Cij, dt, "Cij"),
                                     host_ptr(a_i, dt, "a_i"), host_ptr(a_o, dt, "a_o"), float(taupdt), B, N, M,
                                     host_ptr(weights, dt, "weights"), float(cthr)))
        return Ci, Cj, Cij, weights
    if len(args) == 5:
        weights, Ci, Cj, Cij, cthr = args
        dt = weights.dtype
        N, M = weights.shape
        if Ci.shape != (N,) or Cj.shape != (M,) or Cij.shape != (N, M):
            raise ValueError("update_weights: shape mismatch")
        check(lib.sbb_recompute_weights(dtype_code(dt), host_ptr(weights, dt, "weights"), host_ptr(Ci, dt, "Ci"),
                                        host_ptr(Cj, dt, "Cj"), host_ptr(Cij, dt, "Cij"), float(cthr), N, M))
        return weights
    raise TypeError("update_weights takes 8 (fused) or 5 (un-fused) arguments")


def update_bias(bias, Cj, cthr):
    dt = bias.dtype
    if Cj.shape != bias.shape or bias.ndim != 1:
        raise ValueError("update_bias: shape mismatch")
    check(lib.sbb_update_bias(dtype_code(dt), host_ptr(bias, dt, "bias"), host_ptr(Cj, dt, "Cj"), float(cthr),
                              bias.shape[0]))
    return bias


def update_bias_regularized(bias, kbi, Cj, cthr, khalf, pmin, taubdt):
    dt = bias.dtype
    if Cj.shape != bias.shape or kbi.shape != bias.shape or bias.ndim != 1:
        raise ValueError("update_bias_regularized: shape mismatch")
    check(lib.sbb_update_bias_regularized(dtype_code(dt), host_ptr(bias, dt, "bias"), host_ptr(kbi, dt, "kbi"),
                                          host_ptr(Cj, dt, "Cj"), float(cthr), float(khalf), float(pmin),
                                          float(taubdt), bias.shape[0]))
    return bias, kbi


def update_mask(wmask, weights, Ci, Cj, Cij, cthr, hypercolumns, minicolumns, h, iterations):
    dt = weights.dtype
    code = dtype_code(dt)
    N, M = weights.shape
    if wmask.shape != (N, hypercolumns) or Ci.shape != (N,) or Cj.shape != (M,) or Cij.shape != (N, M):
        raise ValueError("update_mask: shape mismatch")
    check(lib.sbb_update_mask(code, host_ptr(wmask, np.uint8, "wmask"), host_ptr(weights, dt, "weights"),
                              host_ptr(Ci, dt, "Ci"), host_ptr(Cj, dt, "Cj"), host_ptr(Cij, dt, "Cij"), float(cthr),
                              N, M, hypercolumns, minicolumns, int(h), int(iterations)))
    return wmask


def apply_mask(weights, wmask, hypercolumns, minicolumns):
    dt = weights.dtype
    N, M = weights.shape
    if wmask.dtype == np.int8:  # the reference's own test passes int8 (test_openmp.py:243); same bytes
        wmask = wmask.view(np.uint8)
    if wmask.shape != (N, hypercolumns):
        raise ValueError("apply_mask: shape mismatch")
    check(lib.sbb_apply_mask(dtype_code(dt), host_ptr(weights, dt, "weights"), host_ptr(wmask, np.uint8, "wmask"),
                             N, M, hypercolumns, minicolumns))
    return weights


def kernel_launches() -> int:
    return int(lib.sbb_kernel_launches())
