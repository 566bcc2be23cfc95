"""``BCPNN_BACKEND=b200``: the device-resident layer objects and the network driver.

Exports ``Network``, ``DenseLayer`` and ``StructuralPlasticityLayer`` with the
constructor signatures, methods and attributes of the reference's backends
(BCPNN/backend/_cpu_base_backend.py:7-314, specialised as in
BCPNN/backend/cpu_backend.py:7-52).  Differences are confined to where the state
lives: traces, weights, bias, gain and mask stay in HBM inside a C-ABI layer
handle; the attributes ``weights, bias, Ci, Cj, Cij, kbi, wmask`` are properties
that copy device -> host on read and host -> device on assignment.

``compute_activation`` / ``train_step`` accept either numpy arrays (host buffers,
copied in and out by the C ABI) or CUDA ``torch`` tensors (device buffers, no
copies, asynchronous on torch's current stream).

Like the reference's ``cpu`` backend, a structural-plasticity layer always runs 16
swap iterations per mask update whatever ``mask_iterations`` says
(cpu_backend.py:47); pass ``use_mask_iterations=True`` to honour the argument as
the ``numpy``/``gpu`` backends do (_cpu_base_backend.py:154-164).
"""
from __future__ import annotations

import ctypes
from contextlib import nullcontext

import numpy as np

from .. import _lib
from .._lib import STATE, LayerDesc, check, dtype_code, host_ptr, lib
from ..parallel import pipelined_dp_step, sharded_step

try:  # torch is plumbing only: device tensors, streams, torch.distributed
    import torch
except Exception:  # pragma: no cover
    torch = None

__all__ = ["Network", "DenseLayer", "StructuralPlasticityLayer"]


def _is_tensor(a) -> bool:
    return torch is not None and isinstance(a, torch.Tensor)


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _torch_dtype(dtype):
    return torch.float32 if np.dtype(dtype) == np.float32 else torch.float64


class _DeviceLayer:
    """Owns one ``sbb_layer`` handle."""

    _kind = _lib.DENSE
    _state_names = ("weights", "bias", "Ci", "Cj", "Cij")

    def _create(self, dtype, init):
        self.dtype = np.dtype(dtype).type
        desc = LayerDesc(dtype_code(dtype), self._kind, self.in_features, self.hypercolumns, self.minicolumns,
                         float(self.taupdt), float(getattr(self, "khalf", 0.0)), float(getattr(self, "pmin", 0.0)),
                         float(getattr(self, "taubdt", 0.0)), int(self._mask_iterations_used()))
        handle = ctypes.c_void_p()
        check(lib.sbb_layer_create(ctypes.byref(desc), ctypes.byref(handle)))
        self._handle = handle
        self._delta = None
        for name, value in init.items():
            self._set(name, value)

    def _mask_iterations_used(self):
        return 0

    def _shape(self, name):
        N, M, H = self.in_features, self.out_features, self.hypercolumns
        return {"weights": (N, M), "Cij": (N, M), "bias": (M,), "Cj": (M,), "kbi": (M,), "Ci": (N,),
                "wmask": (N, H)}[name]

    def _np_dtype(self, name):
        return np.uint8 if name == "wmask" else self.dtype

    def _get(self, name):
        out = np.empty(self._shape(name), dtype=self._np_dtype(name))
        check(lib.sbb_layer_get_state(self._handle, STATE[name], host_ptr(out), out.nbytes))
        return out

    def _set(self, name, value):
        a = np.ascontiguousarray(np.asarray(value), dtype=self._np_dtype(name))
        if a.shape != self._shape(name):
            raise ValueError("%s must have shape %s, got %s" % (name, self._shape(name), a.shape))
        check(lib.sbb_layer_set_state(self._handle, STATE[name], host_ptr(a), a.nbytes))

    def state_tensor(self, name):
        """A torch view (no copy) of a state array in device memory."""
        ptr = ctypes.c_void_p()
        check(lib.sbb_layer_state_ptr(self._handle, STATE[name], ctypes.byref(ptr)))
        shape = self._shape(name)
        typestr = "|u1" if name == "wmask" else "<f%d" % np.dtype(self.dtype).itemsize
        iface = {"shape": tuple(shape), "typestr": typestr, "data": (ptr.value, False), "version": 2}
        holder = type("_DevicePtr", (), {"__cuda_array_interface__": iface})()
        return torch.as_tensor(holder, device="cuda")

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h is not None and h.value:
            try:
                lib.sbb_layer_destroy(h)
            except Exception:
                pass
            self._handle = None

    # -- reference API ---------------------------------------------------
    def compute_activation(self, inputs):
        """softmax_minicolumns(inputs . weights + bias): _cpu_base_backend.py:44-51, 126-133."""
        B = inputs.shape[0]
        if _is_tensor(inputs):
            x = self._dev_input(inputs, self.in_features)
            y = torch.empty((B, self.out_features), dtype=x.dtype, device=x.device)
            check(lib.sbb_layer_forward(self._handle, x.data_ptr(), B, y.data_ptr(), _stream_ptr()))
            return y
        x = np.ascontiguousarray(inputs, dtype=self.dtype)
        if x.shape[1] != self.in_features:
            raise ValueError("inputs must have %d columns" % self.in_features)
        y = np.empty((B, self.out_features), dtype=self.dtype)
        check(lib.sbb_layer_forward_host(self._handle, host_ptr(x), B, host_ptr(y)))
        return y

    def _dev_input(self, t, cols):
        if not t.is_cuda:
            raise TypeError("torch inputs must be CUDA tensors (pass numpy arrays for host data)")
        if t.dtype != _torch_dtype(self.dtype) or t.dim() != 2 or t.shape[1] != cols:
            raise TypeError("expected a [B, %d] %s tensor" % (cols, np.dtype(self.dtype)))
        return t if t.is_contiguous() else t.contiguous()

    def _train(self, inputs, outputs, h):
        B = inputs.shape[0]
        if _is_tensor(inputs) != _is_tensor(outputs):
            raise TypeError("inputs and outputs must both be numpy arrays or both be CUDA tensors")
        if _is_tensor(inputs):
            x = self._dev_input(inputs, self.in_features)
            y = self._dev_input(outputs, self.out_features)
            check(lib.sbb_layer_train_step(self._handle, x.data_ptr(), y.data_ptr(), B, h, _stream_ptr()))
            return
        x = np.ascontiguousarray(inputs, dtype=self.dtype)
        y = np.ascontiguousarray(outputs, dtype=self.dtype)
        if x.shape[1] != self.in_features or y.shape != (B, self.out_features):
            raise ValueError("train_step: shape mismatch")
        check(lib.sbb_layer_train_step_host(self._handle, host_ptr(x), host_ptr(y), B, h))

    def step_host(self, inputs, targets=None, hypercolumn=None, want_activation=True):
        """Forward + train step from host buffers in ONE call (one upload of the
        inputs): the body of the reference's training loop,
        _cpu_base_backend.py:290-309.  ``targets`` = labels for the classifier,
        None for a hidden layer (which trains on its own activation)."""
        B = inputs.shape[0]
        x = np.ascontiguousarray(inputs, dtype=self.dtype)
        t = None if targets is None else np.ascontiguousarray(targets, dtype=self.dtype)
        y = np.empty((B, self.out_features), dtype=self.dtype) if want_activation else None
        h = -1 if hypercolumn is None else int(hypercolumn)
        check(lib.sbb_layer_step_host(self._handle, host_ptr(x), None if t is None else host_ptr(t), B, h,
                                      None if y is None else host_ptr(y)))
        return y

    def step_host_async(self, inputs, targets=None, hypercolumn=None, out=None):
        """:meth:`step_host` without waiting: the upload of this call's inputs runs beside the
        previous call's step (two staging slots on the device).  ``inputs`` / ``targets`` /
        ``out`` must be C-contiguous arrays of the layer's dtype (page-locked memory for a true
        overlap, e.g. ``torch.empty(...).pin_memory().numpy()``); they may not be touched, and
        ``out`` does not hold the activation, until :meth:`wait` returns."""
        for a in (inputs, targets, out):
            if a is not None and (a.dtype != self.dtype or not a.flags["C_CONTIGUOUS"]):
                raise TypeError("step_host_async needs C-contiguous %s arrays" % np.dtype(self.dtype))
        B = inputs.shape[0]
        if inputs.shape[1] != self.in_features:
            raise ValueError("inputs must have %d columns" % self.in_features)
        for a in (targets, out):
            if a is not None and a.shape != (B, self.out_features):
                raise ValueError("targets / out must be [%d, %d]" % (B, self.out_features))
        h = -1 if hypercolumn is None else int(hypercolumn)
        check(lib.sbb_layer_step_host_async(self._handle, host_ptr(inputs),
                                            None if targets is None else host_ptr(targets), B, h,
                                            None if out is None else host_ptr(out)))

    def wait(self):
        """Block until every :meth:`step_host_async` issued so far has finished."""
        check(lib.sbb_layer_wait(self._handle))

    def train_finalize(self):
        check(lib.sbb_layer_train_finalize(self._handle, _stream_ptr() if torch is not None and
                                           torch.cuda.is_available() else None))

    def convert(self, dtype):
        """Change the precision of the layer (_cpu_base_backend.py:53-59, 135-142)."""
        if np.dtype(dtype) == np.dtype(self.dtype):
            return
        if getattr(self, "_borrowed", False):
            raise RuntimeError("convert() a layer before adding it to a Network")
        state = {n: self._get(n) for n in self._state_names}
        lib.sbb_layer_destroy(self._handle)
        self._handle = None
        self._create(dtype, {n: (v if n == "wmask" else v.astype(dtype)) for n, v in state.items()})

    # -- checkpoint ------------------------------------------------------
    _hyper_names = ("in_features", "hypercolumns", "minicolumns", "taupdt")

    def checkpoint(self) -> dict:
        """State arrays and hyper-parameters as numpy values (see :meth:`Network.save`)."""
        out = {n: self._get(n) for n in self._state_names}
        out["kind"] = np.array(self._kind)
        for n in self._hyper_names:
            out["hp_" + n] = np.array(getattr(self, n))
        return out

    def restore(self, saved: dict) -> None:
        if int(saved["kind"]) != self._kind:
            raise ValueError("checkpoint layer kind %d does not match this layer (%d)" % (int(saved["kind"]), self._kind))
        for n in ("in_features", "hypercolumns", "minicolumns"):
            if int(saved["hp_" + n]) != getattr(self, n):
                raise ValueError("checkpoint %s = %d, this layer has %d" % (n, int(saved["hp_" + n]), getattr(self, n)))
        for n in self._state_names:
            self._set(n, saved[n].astype(self._np_dtype(n)))

    # -- data-parallel step (one exchange: sum of the batch deltas) -------
    def delta_buffer(self):
        if self._delta is None:
            n = int(lib.sbb_layer_delta_elems(self._handle))
            self._delta = torch.empty(n, dtype=_torch_dtype(self.dtype), device="cuda")
        return self._delta

    def dp_train_step(self, inputs, outputs, hypercolumn, world_size, all_reduce, row_blocks=4):
        """Reduce-and-replicate data-parallel train step.  ``all_reduce(tensor)`` must start an in-place
        sum over ranks and return a handle with ``wait()``, e.g. ``dist.all_reduce(t, async_op=True)``;
        every rank reduces and applies the whole matrix
        (:func:`streambrain_b200.parallel.pipelined_dp_step`).  A layer set up by :meth:`shard_rows`
        steps with :meth:`sharded_step` instead (forward and train in one)."""
        if getattr(self, "_shard", None) is not None:
            raise ValueError("the layer is row-sharded: its forward pass and train step run as one sharded_step")
        x = self._dev_input(inputs, self.in_features)
        y = self._dev_input(outputs, self.out_features)
        pipelined_dp_step(_DeviceDPOps(self), x, y, hypercolumn, x.shape[0], world_size, all_reduce, row_blocks)

    # -- row-sharded layer over peer-mapped memory ----------------------------
    def shard_rows(self, rank, world_size, all_gather_bytes, max_local_batch):
        """Give every rank a block of input rows of the layer to own (those rows of the weights, of Cij
        and of Ci).  ``all_gather_bytes(b)`` must return the list of every rank's ``b`` in rank order
        (e.g. through ``torch.distributed.all_gather_object``): it carries the CUDA IPC handles with
        which the ranks map each other's buffers.  ``max_local_batch`` bounds the per-rank batch of
        :meth:`sharded_step`.  One process per GPU, one node, at most 8."""
        n = _lib.SHARD_BUFFERS * _lib.SHARD_HANDLE_BYTES
        mine = (ctypes.c_ubyte * n)()
        check(lib.sbb_layer_shard_init(self._handle, rank, world_size, int(max_local_batch), mine))
        parts = all_gather_bytes(bytes(mine))
        if len(parts) != world_size or any(len(p) != n for p in parts):
            raise ValueError("all_gather_bytes must return one %d-byte string per rank" % n)
        blob = b"".join(parts)
        check(lib.sbb_layer_shard_attach(self._handle, ctypes.c_char_p(blob)))
        self._shard = (rank, world_size)
        self._shard_max_batch = int(max_local_batch)
        self._support = None

    def owned_rows(self, rank=None):
        lo, hi = ctypes.c_long(0), ctypes.c_long(0)
        check(lib.sbb_layer_shard_rows(self._handle, self._shard[0] if rank is None else rank, ctypes.byref(lo),
                                       ctypes.byref(hi)))
        return lo.value, hi.value

    def _barrier_token(self):
        if getattr(self, "_token", None) is None:
            self._token = torch.zeros(1, dtype=torch.float32, device="cuda")
        return self._token

    def sharded_step(self, inputs, hypercolumn, all_reduce, out=None, train=True, next_inputs=None, next_ready=None):
        """Forward pass + train step of an unsupervised layer, row-sharded over the ranks: ``inputs`` is
        this rank's slice of the global batch (the same number of samples on every rank), the return
        value its activations.  ``all_reduce(tensor)`` as in :meth:`dp_train_step`; it sums the supports
        of the global batch and, on a one-element token, serves as the barrier between ranks.  The
        result on every rank's rows equals the single-GPU step at the global batch.  With
        ``train=False`` only the forward pass runs.

        ``next_inputs`` (a device tensor, the slice of the batch the NEXT call will pass as ``inputs``)
        stages that batch ahead: its exchange runs on a side stream beside this step's forward product and
        the step's own all-reduce doubles as its barrier, so the next step starts without one.  The side
        stream waits for the work queued on the current stream so far and for ``next_ready`` (an event,
        e.g. the upload of that batch); :attr:`staged_event` fires when the exchange has read
        ``next_inputs``.  Every rank must make the same choice.  See ``sbb_layer_shard_*`` in the C header for the protocol."""
        x = self._dev_input(inputs, self.in_features)
        xn = None if next_inputs is None else self._dev_input(next_inputs, self.in_features)
        ops = _DeviceShardOps(self, out, next_ready)
        return sharded_step(ops, x, None if hypercolumn is None else int(hypercolumn), all_reduce, xn, train)

    def drop_staged(self):
        """Forget a batch staged by ``next_inputs`` that no step will consume (every rank alike)."""
        if getattr(self, "_staged", None) is not None:
            self._side.synchronize()
            check(lib.sbb_layer_shard_drop_staged(self._handle))
            self._staged = None

    def share_rows(self, all_reduce):
        """While a layer is sharded a rank holds current weights, Cij and Ci only for the rows it owns;
        this copies every owner's rows to all ranks (needed before the plain forward pass, before
        reading the state or writing a checkpoint)."""
        token = self._barrier_token()
        all_reduce(token).wait()
        check(lib.sbb_layer_shard_share_rows(self._handle, _stream_ptr()))
        all_reduce(token).wait()


class _DeviceShardOps:
    """CUDA implementation of the ``ops`` protocol of :func:`streambrain_b200.parallel.sharded_step`."""

    def __init__(self, layer, out, next_ready):
        self.layer, self.out, self.next_ready = layer, out, next_ready
        self.token = layer._barrier_token()
        self.plastic = layer._kind == _lib.PLASTIC
        self.world = layer._shard[1]

    def take_staged(self, x):
        layer = self.layer
        staged = getattr(layer, "_staged", None)
        layer._staged = None
        if staged is None:
            return False
        if staged[0].data_ptr() != x.data_ptr() or staged[0].shape[0] != x.shape[0]:
            layer._staged = staged
            raise ValueError("the previous sharded_step staged another batch as next_inputs; pass that batch, or "
                             "call drop_staged() on every rank")
        return True

    def scatter(self, x, ahead):
        layer = self.layer
        if not ahead:
            check(lib.sbb_layer_shard_scatter(layer._handle, x.data_ptr(), x.shape[0], _stream_ptr()))
            return
        if getattr(layer, "_side", None) is None:
            layer._side = torch.cuda.Stream()
        # the previous step has finished on this rank, so every rank is past the step before it ...
        layer._side.wait_stream(torch.cuda.current_stream())
        if self.next_ready is not None:
            layer._side.wait_event(self.next_ready)
        with torch.cuda.stream(layer._side):
            check(lib.sbb_layer_shard_scatter(layer._handle, x.data_ptr(), x.shape[0], _stream_ptr()))
            layer.staged_event = torch.cuda.Event()
            layer.staged_event.record(layer._side)
        layer._staged = (x,)

    def forward(self, x):
        layer, B = self.layer, x.shape[0]
        if layer._support is None or layer._support.shape[0] != B * self.world:
            layer._support = torch.empty((B * self.world, layer.out_features), dtype=_torch_dtype(layer.dtype),
                                         device="cuda")
        self.B = B
        check(lib.sbb_layer_shard_forward(layer._handle, B, layer._support.data_ptr(), _stream_ptr()))
        return layer._support

    def join_staged(self):
        # ... and this step's all-reduce then certifies that every rank's exchange is complete
        torch.cuda.current_stream().wait_event(self.layer.staged_event)

    def activate(self, support):
        layer = self.layer
        out = self.out
        if out is None:
            out = torch.empty((self.B, layer.out_features), dtype=_torch_dtype(layer.dtype), device="cuda")
        check(lib.sbb_layer_shard_activate(layer._handle, self.B, support.data_ptr(), out.data_ptr(), _stream_ptr()))
        return out

    def train(self, h):
        check(lib.sbb_layer_shard_train(self.layer._handle, self.B, -1 if h is None else h, _stream_ptr()))

    def mask(self, h):
        check(lib.sbb_layer_shard_mask(self.layer._handle, h, _stream_ptr()))


class _DeviceDPOps:
    """CUDA implementation of the ``ops`` protocol of :mod:`streambrain_b200.parallel`."""

    def __init__(self, layer):
        self.layer = layer
        self.delta = layer.delta_buffer()
        self.n_rows, self.n_cols = layer.in_features, layer.out_features

    def local(self, x, y, rb, re):
        check(lib.sbb_layer_dp_local(self.layer._handle, x.data_ptr(), y.data_ptr(), x.shape[0],
                                     self.delta.data_ptr(), rb, re, _stream_ptr()))

    def apply_vectors(self, batch):
        check(lib.sbb_layer_dp_apply_vectors(self.layer._handle, self.delta.data_ptr(), batch, _stream_ptr()))

    def apply_rows(self, batch, rb, re):
        check(lib.sbb_layer_dp_apply_rows(self.layer._handle, self.delta.data_ptr(), batch, rb, re, _stream_ptr()))

    def finish(self, h):
        check(lib.sbb_layer_dp_finish(self.layer._handle, -1 if h is None else int(h), _stream_ptr()))


for _name in ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask"):
    def _getter(self, _n=_name):
        if _n not in self._state_names:
            raise AttributeError(_n)
        return self._get(_n)

    def _setter(self, value, _n=_name):
        if _n not in self._state_names:
            raise AttributeError(_n)
        self._set(_n, value)

    setattr(_DeviceLayer, _name, property(_getter, _setter))


class DenseLayer(_DeviceLayer):
    """Classifier layer: traces and weights every step, bias at ``train_finalize``
    (_cpu_base_backend.py:14-70; cpu_backend.py:13-18).  Initial state follows the
    reference's draw order on the global NumPy stream: randn(N,M) then rand(M)."""

    _kind = _lib.DENSE

    def __init__(self, in_features, hypercolumns, minicolumns, taupdt, initial_counters, dtype=np.float64):
        self.in_features = in_features
        self.hypercolumns = hypercolumns
        self.minicolumns = minicolumns
        self.out_features = hypercolumns * minicolumns
        self.taupdt = taupdt
        N, M = in_features, self.out_features
        init = {
            "weights": (0.1 * np.random.randn(N, M)).astype(dtype),
            "bias": (0.1 * np.random.rand(M)).astype(dtype),
            "Ci": (initial_counters[0] * np.ones([N])).astype(dtype),
            "Cj": (initial_counters[1] * np.ones([M])).astype(dtype),
            "Cij": (initial_counters[2] * np.ones([N, M])).astype(dtype),
        }
        self._create(dtype, init)

    def train_step(self, inputs, outputs):
        self._train(inputs, outputs, -1)


class StructuralPlasticityLayer(_DeviceLayer):
    """Hidden layer with regularised bias and a learned connection mask
    (_cpu_base_backend.py:80-172; cpu_backend.py:29-52).  Draw order:
    randn(N,M), rand(M), rand(N,H) < density."""

    _kind = _lib.PLASTIC
    _state_names = ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask")
    _hyper_names = ("in_features", "hypercolumns", "minicolumns", "taupdt", "khalf", "pmin", "taubdt", "density",
                    "mask_iterations")

    def __init__(self, in_features, hypercolumns, minicolumns, taupdt, khalf, pmin, taubdt, density,
                 mask_iterations, initial_counters, dtype=np.float64, use_mask_iterations=False):
        self.in_features = in_features
        self.hypercolumns = hypercolumns
        self.minicolumns = minicolumns
        self.out_features = hypercolumns * minicolumns
        self.taupdt = taupdt
        self.khalf = khalf
        self.pmin = pmin
        self.taubdt = taubdt
        self.density = density
        self.mask_iterations = mask_iterations
        self.use_mask_iterations = use_mask_iterations
        N, M = in_features, self.out_features
        init = {
            "weights": (0.1 * np.random.randn(N, M)).astype(dtype),
            "bias": (0.1 * np.random.rand(M)).astype(dtype),
            "Ci": (initial_counters[0] * np.ones([N])).astype(dtype),
            "Cj": (initial_counters[1] * np.ones([M])).astype(dtype),
            "Cij": (initial_counters[2] * np.ones([N, M])).astype(dtype),
            "kbi": np.ones([M]).astype(dtype),
        }
        init["wmask"] = (np.random.rand(N, hypercolumns) < density).astype(np.uint8)
        self._create(dtype, init)

    def _mask_iterations_used(self):
        return self.mask_iterations if self.use_mask_iterations else 16

    def train_step(self, inputs, outputs, hypercolumn=None):
        self._train(inputs, outputs, -1 if hypercolumn is None else int(hypercolumn))


class Network:
    """Layer container with the reference's ``fit`` / ``evaluate`` interface
    (_cpu_base_backend.py:174-245) on top of the native loop driver (``sbb_network_*``).

    The loops themselves run in the C library: the dataset is uploaded once per call, every batch is
    assembled on the device from the epoch's sample order, and nothing synchronises with the host until
    an epoch (or an evaluation) ends.  What stays here is what must come from Python to reproduce a
    seeded reference run: per epoch one permutation of the samples and then one of the trained layer's
    hypercolumns, both drawn from NumPy's global stream (_cpu_base_backend.py:258-264).

    With ``world_size > 1`` every rank takes the reference's slice of each batch
    (_cpu_base_backend.py:279-288) and, when :meth:`set_data_parallel` was given ``all_reduce``, the
    trained layer sums its batch deltas over the ranks once per step (the mpi backend's scheme).
    """

    CHUNK = 64   # batches queued per native call: the granularity of the progress bar
    verbose = True

    def __init__(self, dtype):
        self.dtype = dtype
        self._layers = []
        self.world_rank = 0
        self.world_size = 1
        self._all_reduce = None
        self._sum_counts = None
        self._all_gather_bytes = None
        self._handle = ctypes.c_void_p()
        check(lib.sbb_network_create(dtype_code(dtype), ctypes.byref(self._handle)))
        self._comm = None
        self._pending = {}

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h is not None and h.value:
            try:
                lib.sbb_network_destroy(h)
            except Exception:
                pass
            self._handle = None

    # -- data parallelism ---------------------------------------------------
    def set_data_parallel(self, rank, world_size, all_reduce=None, sum_counts=None, all_gather_bytes=None):
        """``all_reduce(tensor) -> handle with wait()`` starts an in-place sum of a device tensor over
        the ranks (``dist.all_reduce(t, async_op=True)``); ``sum_counts(np.ndarray) -> np.ndarray`` sums
        the evaluation counters (the mpi backend's Allreduce, mpi_backend.py:63-69).  With
        ``all_gather_bytes`` (see :meth:`_DeviceLayer.shard_rows`) the layers that learn from their own
        activations (all but the last) are row-sharded over the ranks when :meth:`fit` first trains them
        and step with the sharded step instead of reduce-and-replicate."""
        self.world_rank, self.world_size = rank, world_size
        self._all_reduce, self._sum_counts = all_reduce, sum_counts
        self._all_gather_bytes = all_gather_bytes
        comm = None
        if all_reduce is not None:
            comm = self._make_comm(all_reduce)
        self._comm = comm   # keeps the callbacks alive
        check(lib.sbb_network_set_data_parallel(self._handle, rank, world_size,
                                                ctypes.byref(comm) if comm is not None else None))

    def _make_comm(self, all_reduce):
        pending = self._pending
        tdtype = {_lib.F32: torch.float32, _lib.F64: torch.float64}
        ticket = [0]

        def begin(_user, ptr, elems, dtype, stream):
            try:
                typestr = "<f4" if dtype == _lib.F32 else "<f8"
                holder = type("_DevicePtr", (), {"__cuda_array_interface__": {
                    "shape": (int(elems),), "typestr": typestr, "data": (int(ptr), False), "version": 2}})()
                with torch.cuda.stream(torch.cuda.ExternalStream(int(stream or 0))):
                    t = torch.as_tensor(holder, device="cuda")
                    assert t.dtype == tdtype[dtype]
                    work = all_reduce(t)
                ticket[0] += 1
                pending[ticket[0]] = (work, t)
                return ticket[0]
            except Exception:   # an exception must not unwind through the C caller
                import traceback
                traceback.print_exc()
                return -1

        def wait(_user, token, stream):
            try:
                work, _t = pending.pop(int(token))
                with torch.cuda.stream(torch.cuda.ExternalStream(int(stream or 0))):
                    work.wait()
                return 0
            except Exception:
                import traceback
                traceback.print_exc()
                return 1

        return _lib.Comm(None, _lib.REDUCE_BEGIN_FN(begin), _lib.REDUCE_WAIT_FN(wait))

    # -- reference API --------------------------------------------------------
    def add_layer(self, layer):
        if layer.dtype != self.dtype:
            layer.convert(self.dtype)
        check(lib.sbb_network_add_layer(self._handle, layer._handle))
        self._layers.append(layer)
        layer._borrowed = True   # the network holds the native handle: it must not be re-created

    def _upload(self, data, labels):
        x = np.ascontiguousarray(data, dtype=self.dtype)
        t = np.ascontiguousarray(labels, dtype=self.dtype)
        if x.ndim != 2 or t.ndim != 2 or x.shape[0] != t.shape[0]:
            raise ValueError("data and labels must be [n, features] and [n, classes]")
        check(lib.sbb_network_set_dataset(self._handle, host_ptr(x), host_ptr(t), x.shape[0], x.shape[1], t.shape[1]))
        return x.shape[0]

    def _progress(self, total, description):
        if self.world_rank == 0 and self.verbose:
            from tqdm import tqdm
            bar = tqdm(total=total)
            bar.set_description(description)
            return bar
        return nullcontext()

    def fit(self, training_data, training_labels, maximal_batch_size, schedule):
        """_cpu_base_backend.py:188-203, 247-314."""
        n = self._upload(training_data, training_labels)
        batches = (n + maximal_batch_size - 1) // maximal_batch_size
        for layer, epochs in schedule:
            hypercolumns = self._layers[layer].hypercolumns
            target = self._layers[layer]
            if (self._all_gather_bytes is not None and layer + 1 < len(self._layers)
                    and getattr(target, "_shard", None) is None):
                # every rank takes floor(batch / world_size) samples of a batch (sbb_network_batch_plan)
                target.shard_rows(self.world_rank, self.world_size, self._all_gather_bytes,
                                  max(1, maximal_batch_size // self.world_size))
            if (getattr(target, "_shard", None) is not None and layer + 1 < len(self._layers)
                    and maximal_batch_size // self.world_size > target._shard_max_batch):
                raise ValueError("layer %d was sharded for local batches of up to %d samples; this fit needs %d" % (
                    layer, target._shard_max_batch, maximal_batch_size // self.world_size))
            for epoch in range(epochs):
                if self.world_rank == 0 and self.verbose:
                    print('Layer - %d/%d' % (layer + 1, len(self._layers)), flush=True)
                # the two draws of an epoch, in the reference's order
                order = np.ascontiguousarray(np.random.permutation(range(n)), dtype=np.int64)
                hc_order = np.ascontiguousarray(np.random.permutation(range(hypercolumns)), dtype=np.int64)
                check(lib.sbb_network_set_epoch_order(self._handle, host_ptr(order)))
                with self._progress(batches, 'Epoch %d/%d' % (epoch + 1, epochs)) as bar:
                    for first in range(0, batches, self.CHUNK):
                        upto = min(batches, first + self.CHUNK)
                        rc = lib.sbb_network_train_batches(self._handle, layer, maximal_batch_size, host_ptr(hc_order),
                                                           epoch, first, upto)
                        if rc == _lib.ERR_UNSUPPORTED and b"division by zero" in (lib.sbb_last_error() or b""):
                            # fewer batches than hypercolumns + 1: the reference fails in `i % (nb // (H + 1))`
                            raise ZeroDivisionError(lib.sbb_last_error().decode())
                        check(rc)
                        if bar is not None:
                            bar.update(upto - first)

    def evaluate(self, images, labels, maximal_batch_size):
        """_cpu_base_backend.py:205-245: (correct, total) as one-element arrays."""
        self._upload(images, labels)
        hit, seen = ctypes.c_long(0), ctypes.c_long(0)
        with self._progress(1, "Evaluation") as bar:
            check(lib.sbb_network_evaluate(self._handle, maximal_batch_size, ctypes.byref(hit), ctypes.byref(seen)))
            if bar is not None:
                bar.update(1)
        correct, total = np.array([hit.value]), np.array([seen.value])
        if self.world_size > 1 and self._sum_counts is not None:
            correct, total = self._sum_counts(correct), self._sum_counts(total)
        return correct, total

    # -- checkpoint / resume ----------------------------------------------------
    def save(self, path):
        """Write every layer's state arrays and hyper-parameters to one ``.npz`` file.  The reference has
        no checkpointing (its only trace dump is commented out: full_cuda_backend/debug_dump.cpp:1-22)."""
        blob = {"n_layers": np.array(len(self._layers)), "dtype": np.array(np.dtype(self.dtype).str)}
        for k, layer in enumerate(self._layers):
            for name, value in layer.checkpoint().items():
                blob["l%d_%s" % (k, name)] = value
        np.savez(path, **blob)

    def load(self, path):
        """Restore the state written by :meth:`save` into this network's layers (same layer kinds and
        shapes).  Training resumed after ``load`` continues exactly as the saved run would have."""
        with np.load(path) as z:
            if int(z["n_layers"]) != len(self._layers):
                raise ValueError("checkpoint holds %d layers, the network has %d" % (int(z["n_layers"]),
                                                                                    len(self._layers)))
            for k, layer in enumerate(self._layers):
                prefix = "l%d_" % k
                layer.restore({n[len(prefix):]: z[n] for n in z.files if n.startswith(prefix)})
