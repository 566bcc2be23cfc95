"""ctypes binding of libsbb200.so (the C ABI declared in include/sbb200.h).

The library is the only compute path of this package: if it cannot be loaded the
import raises, and every compute call raises :class:`SbbError` when the library
reports a failure (including "no CUDA device").  There is no CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_long, c_size_t, c_ulonglong, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# SBB_LIBRARY points at an alternative build of the same library (e.g. one with extra diagnostics).
LIB_PATH = os.environ.get("SBB_LIBRARY") or os.path.join(HERE, "libsbb200.so")

SBB_OK = 0
ERR_NAMES = {1: "SBB_ERR_INVALID", 2: "SBB_ERR_CUDA", 3: "SBB_ERR_NO_DEVICE", 4: "SBB_ERR_UNSUPPORTED",
             5: "SBB_ERR_TIMEOUT"}
ERR_INVALID, ERR_CUDA, ERR_NO_DEVICE, ERR_UNSUPPORTED, ERR_TIMEOUT = 1, 2, 3, 4, 5
F32, F64 = 0, 1
SHARD_BUFFERS, SHARD_HANDLE_BYTES = 7, 64
DENSE, PLASTIC = 0, 1
STATE = {"weights": 0, "bias": 1, "Ci": 2, "Cj": 3, "Cij": 4, "kbi": 5, "wmask": 6}


class SbbError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("%s: %s" % (ERR_NAMES.get(code, "error %d" % code), message))
        self.code = code


class LayerDesc(ctypes.Structure):
    _fields_ = [("dtype", c_int), ("kind", c_int), ("in_features", c_long), ("hypercolumns", c_long),
                ("minicolumns", c_long), ("taupdt", c_double), ("khalf", c_double), ("pmin", c_double),
                ("taubdt", c_double), ("mask_iterations", c_long)]


REDUCE_BEGIN_FN = ctypes.CFUNCTYPE(c_long, c_void_p, c_void_p, c_size_t, c_int, c_void_p)
REDUCE_WAIT_FN = ctypes.CFUNCTYPE(c_int, c_void_p, c_long, c_void_p)


class Comm(ctypes.Structure):
    """``sbb_comm``: how a data-parallel network sums device buffers over ranks."""
    _fields_ = [("user", c_void_p), ("reduce_begin", REDUCE_BEGIN_FN), ("reduce_wait", REDUCE_WAIT_FN)]


# name -> (restype, argtypes); one entry per declaration in include/sbb200.h
SIGNATURES = {
    "sbb_version": (c_int, []),
    "sbb_last_error": (c_char_p, []),
    "sbb_device_count": (c_int, []),
    "sbb_update_state": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_long, c_long]),
    "sbb_add_bias": (c_int, [c_int, c_void_p, c_void_p, c_long, c_long]),
    "sbb_softmax_minicolumns": (c_int, [c_int, c_void_p, c_long, c_long, c_long]),
    "sbb_update_counters": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_double, c_long,
                                    c_long, c_long]),
    "sbb_update_weights": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_double, c_long,
                                   c_long, c_long, c_void_p, c_double]),
    "sbb_recompute_weights": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_double, c_long, c_long]),
    "sbb_update_bias": (c_int, [c_int, c_void_p, c_void_p, c_double, c_long]),
    "sbb_update_bias_regularized": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_double, c_double, c_double,
                                            c_double, c_long]),
    "sbb_update_mask": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_double, c_long, c_long,
                                c_long, c_long, c_long, c_long]),
    "sbb_apply_mask": (c_int, [c_int, c_void_p, c_void_p, c_long, c_long, c_long, c_long]),
    "sbb_layer_create": (c_int, [POINTER(LayerDesc), POINTER(c_void_p)]),
    "sbb_layer_destroy": (c_int, [c_void_p]),
    "sbb_layer_set_state": (c_int, [c_void_p, c_int, c_void_p, c_size_t]),
    "sbb_layer_get_state": (c_int, [c_void_p, c_int, c_void_p, c_size_t]),
    "sbb_layer_state_ptr": (c_int, [c_void_p, c_int, POINTER(c_void_p)]),
    "sbb_layer_forward": (c_int, [c_void_p, c_void_p, c_long, c_void_p, c_void_p]),
    "sbb_layer_train_step": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long, c_void_p]),
    "sbb_layer_train_finalize": (c_int, [c_void_p, c_void_p]),
    "sbb_layer_forward_host": (c_int, [c_void_p, c_void_p, c_long, c_void_p]),
    "sbb_layer_train_step_host": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long]),
    "sbb_layer_step_host": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long, c_void_p]),
    "sbb_layer_delta_elems": (c_size_t, [c_void_p]),
    "sbb_layer_dp_local": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_long, c_long, c_void_p]),
    "sbb_layer_dp_apply_vectors": (c_int, [c_void_p, c_void_p, c_long, c_void_p]),
    "sbb_layer_dp_apply_rows": (c_int, [c_void_p, c_void_p, c_long, c_long, c_long, c_void_p]),
    "sbb_layer_dp_finish": (c_int, [c_void_p, c_long, c_void_p]),
    "sbb_layer_info": (c_int, [c_void_p, POINTER(LayerDesc)]),
    "sbb_network_batch_plan": (c_int, [c_long, c_long, c_long, c_long, c_long, c_long, c_long, POINTER(c_long),
                                       POINTER(c_long), POINTER(c_long)]),
    "sbb_network_create": (c_int, [c_int, POINTER(c_void_p)]),
    "sbb_network_destroy": (c_int, [c_void_p]),
    "sbb_network_add_layer": (c_int, [c_void_p, c_void_p]),
    "sbb_network_set_data_parallel": (c_int, [c_void_p, c_long, c_long, c_void_p]),
    "sbb_network_set_dataset": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long, c_long]),
    "sbb_network_set_epoch_order": (c_int, [c_void_p, c_void_p]),
    "sbb_network_train_batches": (c_int, [c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_long]),
    "sbb_network_evaluate": (c_int, [c_void_p, c_long, POINTER(c_long), POINTER(c_long)]),
    "sbb_layer_shard_init": (c_int, [c_void_p, c_long, c_long, c_long, c_void_p]),
    "sbb_layer_shard_attach": (c_int, [c_void_p, c_void_p]),
    "sbb_layer_shard_scatter": (c_int, [c_void_p, c_void_p, c_long, c_void_p]),
    "sbb_layer_shard_forward": (c_int, [c_void_p, c_long, c_void_p, c_void_p]),
    "sbb_layer_shard_activate": (c_int, [c_void_p, c_long, c_void_p, c_void_p, c_void_p]),
    "sbb_layer_shard_train": (c_int, [c_void_p, c_long, c_long, c_void_p]),
    "sbb_layer_shard_mask": (c_int, [c_void_p, c_long, c_void_p]),
    "sbb_layer_shard_share_rows": (c_int, [c_void_p, c_void_p]),
    "sbb_layer_shard_drop_staged": (c_int, [c_void_p]),
    "sbb_layer_shard_world": (c_long, [c_void_p]),
    "sbb_layer_shard_rows": (c_int, [c_void_p, c_long, POINTER(c_long), POINTER(c_long)]),
    "sbb_count_correct": (c_int, [c_int, c_void_p, c_void_p, c_long, c_long, POINTER(c_long), c_void_p]),
    "sbb_update_mask_noalloc": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_double, c_long,
                                        c_long, c_long, c_long, c_long, c_long, c_void_p]),
    "sbb_noalloc_last_error": (c_char_p, []),
    "sbb_layer_profile": (c_int, [c_void_p, c_int]),
    "sbb_layer_phase_calls": (c_int, [c_void_p, c_int, POINTER(c_long)]),
    "sbb_layer_phase_ms": (c_int, [c_void_p, c_int, c_long, POINTER(ctypes.c_float)]),
    "sbb_set_contraction_path": (c_int, [c_int]),
    "sbb_get_contraction_path": (c_int, []),
    "sbb_layer_step_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long, c_void_p]),
    "sbb_layer_wait": (c_int, [c_void_p]),
    "sbb_set_reserved_sms": (c_int, [c_int]),
    "sbb_get_reserved_sms": (c_int, []),
    "sbb_tensor_path_available": (c_int, []),
    "sbb_device_wait_status": (c_int, [POINTER(c_int)]),
    "sbb_device_clear_wait_status": (c_int, []),
    "sbb_set_wait_limit_cycles": (c_int, [ctypes.c_longlong]),
    "sbb_get_wait_limit_cycles": (ctypes.c_longlong, []),
    "sbb_debug_lose_arrival": (c_int, [c_int]),
    "sbb_idx_info": (c_int, [c_char_p, POINTER(c_int), POINTER(c_long)]),
    "sbb_read_idx_images": (c_int, [c_char_p, c_int, c_void_p, c_long, c_long]),
    "sbb_read_idx_labels": (c_int, [c_char_p, c_int, c_void_p, c_long, c_long]),
    "sbb_raw_u8_count": (c_int, [c_char_p, POINTER(c_long)]),
    "sbb_read_raw_u8_images": (c_int, [c_char_p, c_int, c_void_p, c_long, c_long]),
    "sbb_read_raw_u8_labels": (c_int, [c_char_p, c_int, c_void_p, c_long, c_long, c_long]),
    "sbb_measure_fp64_rates": (c_int, [POINTER(c_double), POINTER(c_double)]),
    "sbb_kernel_launches": (c_ulonglong, []),
    "sbb_stream_sync": (c_int, [c_void_p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: build it with `python -m streambrain_b200.build` "
                          "(there is no CPU fallback)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != SBB_OK:
        raise SbbError(rc, (lib.sbb_last_error() or b"").decode("utf-8", "replace"))


def dtype_code(dtype) -> int:
    dt = np.dtype(dtype)
    if dt == np.float32:
        return F32
    if dt == np.float64:
        return F64
    raise Exception("Invalid dtype")


def host_ptr(a: np.ndarray, dtype=None, name="array") -> c_void_p:
    """Pointer to a numpy array the native side may mutate in place.  Unlike
    pybind11's implicit conversion this never copies: a wrong dtype or a
    non-contiguous array is an error."""
    if not isinstance(a, np.ndarray):
        raise TypeError("%s must be a numpy array" % name)
    if dtype is not None and a.dtype != np.dtype(dtype):
        raise TypeError("%s has dtype %s, expected %s" % (name, a.dtype, np.dtype(dtype)))
    if not a.flags["C_CONTIGUOUS"]:
        raise TypeError("%s must be C-contiguous" % name)
    return c_void_p(a.ctypes.data)
