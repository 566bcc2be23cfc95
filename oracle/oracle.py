"""CPU oracle for the BCPNN layer train step -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may
import this module; the shipped package never does.  Two interchangeable kernel
sets expose the kernel-wrapper interface of StreamBrain's
``BCPNN/backend/_kernels/kernels_openmp.py:6-99`` (same names, argument order,
in-place mutation, returned arrays):

* :class:`PortKernels`   -- our plain-C restatement (``bcpnn_oracle.c``), via ctypes.
* :class:`RefKernels`    -- StreamBrain's own compiled OpenMP module
  (``oracle/_ref``, built by ``oracle/build.py`` from the reference checkout),
  with the NumPy softmax the ``cpu`` backend uses (``cpu_backend.py:10,24``).

:class:`OracleLayer` restates the layer objects and the step order of the ``cpu``
backend (``BCPNN/backend/cpu_backend.py:7-52`` over
``BCPNN/backend/_cpu_base_backend.py:7-172``) on top of either kernel set.
"""
from __future__ import annotations

import ctypes
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)
import build as _build  # noqa: E402  (oracle/build.py)

_c_long = ctypes.c_long
_SUFFIX = {np.dtype(np.float32): "_f32", np.dtype(np.float64): "_f64"}


def _check(a, dtype=None):
    if not isinstance(a, np.ndarray) or not a.flags["C_CONTIGUOUS"]:
        raise TypeError("oracle expects C-contiguous numpy arrays")
    if dtype is not None and a.dtype != dtype:
        raise TypeError("oracle dtype mismatch: %s vs %s" % (a.dtype, dtype))
    return a.ctypes.data_as(ctypes.c_void_p)


def numpy_softmax_minicolumns(a, hypercolumns, minicolumns):
    """BCPNN/backend/_kernels/kernels_numpy.py:13-25."""
    v = np.reshape(a, [-1, hypercolumns, minicolumns])
    t = np.exp(v - v.max(axis=2, keepdims=True))
    return np.reshape(t / np.sum(t, axis=2, keepdims=True), [-1, hypercolumns * minicolumns])


class PortKernels:
    """ctypes view of libbcpnn_oracle.so (kind = "port")."""

    kind = "port"

    def __init__(self):
        self.lib = ctypes.CDLL(_build.build_oracle())

    def _fn(self, name, dtype, restype=None):
        f = getattr(self.lib, name + _SUFFIX[np.dtype(dtype)])
        f.restype = restype
        return f

    @staticmethod
    def _real(dtype):
        return ctypes.c_float if np.dtype(dtype) == np.float32 else ctypes.c_double

    def update_state(self, state, weights, bias, inputs):
        dt = state.dtype
        B, N = inputs.shape
        M = weights.shape[1]
        if weights.shape[0] != N or state.shape != (B, M) or bias.shape != (M,):
            raise ValueError("update_state: shape mismatch")
        self._fn("orc_update_state", dt)(_check(state, dt), _check(inputs, dt), _check(weights, dt),
                                         _check(bias, dt), _c_long(B), _c_long(N), _c_long(M))
        return state

    def softmax_minicolumns(self, a, hypercolumns, minicolumns):
        dt = a.dtype
        rows = a.size // (hypercolumns * minicolumns)
        self._fn("orc_softmax_minicolumns", dt)(_check(a, dt), _c_long(rows), _c_long(hypercolumns),
                                                _c_long(minicolumns))
        return a

    def update_weights(self, Ci, Cj, Cij, a_i, a_o, taupdt, weights, cthr):
        dt = Ci.dtype
        R = self._real(dt)
        B, N = a_i.shape
        M = a_o.shape[1]
        if Ci.shape != (N,) or Cj.shape != (M,) or Cij.shape != (N, M) or weights.shape != (N, M) \
                or a_o.shape[0] != B:
            raise ValueError("update_weights: shape mismatch")
        self._fn("orc_update_weights", dt, R)(R(1.0), _check(Ci, dt), _check(Cj, dt), _check(Cij, dt),
                                              _check(a_i, dt), _check(a_o, dt), R(taupdt), _c_long(B),
                                              _c_long(N), _c_long(M), _check(weights, dt), R(cthr))
        return Ci, Cj, Cij, weights

    def update_counters(self, Ci, Cj, Cij, a_i, a_o, taupdt):
        dt = Ci.dtype
        R = self._real(dt)
        B, N = a_i.shape
        M = a_o.shape[1]
        if Ci.shape != (N,) or Cj.shape != (M,) or Cij.shape != (N, M) or a_o.shape[0] != B:
            raise ValueError("update_counters: shape mismatch")
        self._fn("orc_update_counters", dt)(_check(Ci, dt), _check(Cj, dt), _check(Cij, dt),
                                            _check(a_i, dt), _check(a_o, dt), R(taupdt), _c_long(B),
                                            _c_long(N), _c_long(M))
        return Ci, Cj, Cij

    def recompute_weights(self, weights, Ci, Cj, Cij, cthr):
        dt = weights.dtype
        R = self._real(dt)
        N, M = weights.shape
        self._fn("orc_recompute_weights", dt)(_check(weights, dt), _check(Ci, dt), _check(Cj, dt),
                                              _check(Cij, dt), R(cthr), _c_long(N), _c_long(M))
        return weights

    def update_bias(self, bias, Cj, cthr):
        dt = bias.dtype
        R = self._real(dt)
        self._fn("orc_update_bias", dt)(_check(bias, dt), _check(Cj, dt), R(cthr), _c_long(bias.shape[0]))
        return bias

    def update_bias_regularized(self, bias, kbi, Cj, cthr, khalf, pmin, taubdt):
        dt = bias.dtype
        R = self._real(dt)
        self._fn("orc_update_bias_regularized", dt)(_check(bias, dt), _check(kbi, dt), _check(Cj, dt),
                                                    R(cthr), R(khalf), R(pmin), R(taubdt),
                                                    _c_long(bias.shape[0]))
        return bias, kbi

    def update_mask(self, wmask, weights, Ci, Cj, Cij, cthr, hypercolumns, minicolumns, h, iterations):
        dt = weights.dtype
        R = self._real(dt)
        N, M = weights.shape
        if M != hypercolumns * minicolumns or wmask.shape != (N, hypercolumns) or Cij.shape != (N, M) \
                or Ci.shape != (N,) or Cj.shape != (M,) or not 0 <= h < hypercolumns:
            raise ValueError("update_mask: shape mismatch")
        self._fn("orc_update_mask", dt)(_check(wmask, np.uint8), _check(weights, dt), _check(Ci, dt),
                                        _check(Cj, dt), _check(Cij, dt), R(cthr), _c_long(N), _c_long(M),
                                        _c_long(h), _c_long(hypercolumns), _c_long(minicolumns),
                                        _c_long(iterations))
        return wmask

    def apply_mask(self, weights, wmask, hypercolumns, minicolumns):
        dt = weights.dtype
        N, M = weights.shape
        if M != hypercolumns * minicolumns or wmask.shape != (N, hypercolumns):
            raise ValueError("apply_mask: shape mismatch")
        self._fn("orc_apply_mask", dt)(_check(weights, dt), _check(wmask, np.uint8), _c_long(N),
                                       _c_long(M), _c_long(hypercolumns), _c_long(minicolumns))
        return weights


def ref_available() -> bool:
    path = _build.ref_module_path()
    return os.path.exists(path) or _build.reference_root() is not None


class RefKernels:
    """StreamBrain's compiled OpenMP kernel module (kind = "reference").

    The dtype dispatch restates BCPNN/backend/_kernels/kernels_openmp.py:6-99; the
    native functions are the reference's own (kernels_openmp_internal.cc:460-478).
    """

    kind = "reference"

    def __init__(self):
        path = _build.build_reference()
        if path is None or not os.path.exists(path):
            raise RuntimeError("compiled reference module not available (oracle/_ref is empty)")
        spec = importlib.util.spec_from_file_location(_build.REF_MODULE_NAME, path)
        self._i = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(self._i)
        self.path = path

    def _f(self, name, dtype):
        if dtype == np.float64:
            return getattr(self._i, name + "_float64")
        if dtype == np.float32:
            return getattr(self._i, name + "_float32")
        raise Exception("Invalid dtype")

    def update_state(self, state, weights, bias, inputs):
        self._f("update_state", state.dtype)(state, inputs, weights, bias)
        return state

    def softmax_minicolumns(self, a, hypercolumns, minicolumns):
        return numpy_softmax_minicolumns(a, hypercolumns, minicolumns)

    def update_weights(self, Ci, Cj, Cij, a_i, a_o, taupdt, weights, cthr):
        self._f("update_weights", Ci.dtype)(1.0, Ci, Cj, Cij, a_i, a_o, taupdt, weights, cthr)
        return Ci, Cj, Cij, weights

    def update_bias(self, bias, Cj, cthr):
        self._f("update_bias", bias.dtype)(bias, Cj, cthr)
        return bias

    def update_bias_regularized(self, bias, kbi, Cj, cthr, khalf, pmin, taubdt):
        self._f("update_bias_regularized", bias.dtype)(bias, kbi, Cj, cthr, khalf, pmin, taubdt)
        return bias, kbi

    def update_mask(self, wmask, weights, Ci, Cj, Cij, cthr, hypercolumns, minicolumns, h, iterations):
        self._f("update_mask", weights.dtype)(wmask, weights, Ci, Cj, Cij, cthr, hypercolumns,
                                              minicolumns, h, iterations)
        return wmask

    def apply_mask(self, weights, wmask, hypercolumns, minicolumns):
        self._f("apply_mask", weights.dtype)(weights, wmask, hypercolumns, minicolumns)
        return weights


class OracleLayer:
    """A BCPNN layer of the reference's ``cpu`` backend, on host numpy state.

    ``kind="plastic"``: StructuralPlasticityLayer (_cpu_base_backend.py:80-172 with
    the fused train_step of cpu_backend.py:29-52).  ``kind="dense"``: DenseLayer
    (_cpu_base_backend.py:14-70, cpu_backend.py:13-18).  Initial state follows the
    constructor's RNG order: randn(N,M) -> rand(M) -> rand(N,H) on ``rng``
    (_cpu_base_backend.py:31-42, :107-124).
    """

    def __init__(self, kernels, kind, in_features, hypercolumns, minicolumns, taupdt,
                 initial_counters, dtype, khalf=0.0, pmin=0.0, taubdt=0.0, density=1.0, rng=None):
        rng = rng if rng is not None else np.random
        self.k = kernels
        self.kind = kind
        self.in_features, self.hypercolumns, self.minicolumns = in_features, hypercolumns, minicolumns
        self.out_features = hypercolumns * minicolumns
        self.taupdt, self.khalf, self.pmin, self.taubdt, self.density = taupdt, khalf, pmin, taubdt, density
        self.dtype = np.dtype(dtype)
        N, M = in_features, self.out_features
        self.weights = (0.1 * rng.randn(N, M)).astype(dtype)
        self.bias = (0.1 * rng.rand(M)).astype(dtype)
        self.Ci = (initial_counters[0] * np.ones([N])).astype(dtype)
        self.Cj = (initial_counters[1] * np.ones([M])).astype(dtype)
        self.Cij = (initial_counters[2] * np.ones([N, M])).astype(dtype)
        if kind == "plastic":
            self.kbi = np.ones([M]).astype(dtype)
            self.wmask = (rng.rand(N, hypercolumns) < density).astype(np.uint8)

    def state(self):
        names = ["weights", "bias", "Ci", "Cj", "Cij"] + (["kbi", "wmask"] if self.kind == "plastic" else [])
        return {n: getattr(self, n).copy() for n in names}

    def compute_activation(self, inputs):
        """_cpu_base_backend.py:44-51 / :126-133."""
        act = np.zeros([inputs.shape[0], self.out_features], dtype=self.dtype)
        act = self.k.update_state(act, self.weights, self.bias, np.ascontiguousarray(inputs))
        return self.k.softmax_minicolumns(act, self.hypercolumns, self.minicolumns)

    def train_step(self, inputs, outputs, hypercolumn=None):
        """cpu_backend.py:13-15 (dense) / :29-52 (plastic; mask iterations fixed at 16)."""
        cthr = self.taupdt / 2
        self.Ci, self.Cj, self.Cij, self.weights = self.k.update_weights(
            self.Ci, self.Cj, self.Cij, np.ascontiguousarray(inputs), np.ascontiguousarray(outputs),
            self.taupdt, self.weights, cthr)
        if self.kind != "plastic":
            return
        self.bias, self.kbi = self.k.update_bias_regularized(
            self.bias, self.kbi, self.Cj, cthr, self.khalf, self.pmin, self.taubdt)
        if hypercolumn is not None:
            self.wmask = self.k.update_mask(self.wmask, self.weights, self.Ci, self.Cj, self.Cij, cthr,
                                            self.hypercolumns, self.minicolumns, int(hypercolumn), 16)
        self.weights = self.k.apply_mask(self.weights, self.wmask, self.hypercolumns, self.minicolumns)

    def train_finalize(self):
        """cpu_backend.py:17-18 (dense) / _cpu_base_backend.py:171-172 (plastic: no-op)."""
        if self.kind == "dense":
            self.bias = self.k.update_bias(self.bias, self.Cj, self.taupdt / 2)


def best_kernels():
    """The compiled reference when present, else the port."""
    try:
        return RefKernels()
    except Exception:
        return PortKernels()
