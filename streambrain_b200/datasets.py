"""Readers for the dataset files the reference's training driver consumes.

Function names and results follow StreamBrain's ``train.py:9-41``:

* ``load_mnist(image_file, label_file, dtype)`` -- IDX image / label files (MNIST and
  Fashion-MNIST): images as ``[n, rows*cols]`` scaled to [0, 1], labels as one-hot ``[n, 10]``;
* ``load_stl_10_images(file)`` -- headerless bytes, ``[n, 3*96*96]`` in file order, scaled to [0, 1];
* ``load_stl_10_labels(file)`` -- bytes 1..10 as one-hot ``[n, 10]``.

The parsing runs in the C library (``sbb_read_idx_*``, ``sbb_read_raw_u8_*``), which -- unlike the
reference, which skips 16 / 8 header bytes unchecked (train.py:10-18) -- validates the IDX magic, rank
and element type and the sizes against the file, and raises instead of mis-reading.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from ._lib import check, dtype_code, host_ptr, lib

STL10_FEATURES = 3 * 96 * 96


def idx_shape(path) -> tuple:
    """Dimensions recorded in an IDX file's header."""
    ndim = ctypes.c_int(0)
    dims = (ctypes.c_long * 4)()
    check(lib.sbb_idx_info(os.fsencode(path), ctypes.byref(ndim), dims))
    return tuple(int(dims[d]) for d in range(ndim.value))


def read_idx_images(path, dtype=np.float64) -> np.ndarray:
    shape = idx_shape(path)
    n = shape[0]
    features = int(np.prod(shape[1:])) if len(shape) > 1 else 1
    out = np.empty((n, features), dtype=dtype)
    check(lib.sbb_read_idx_images(os.fsencode(path), dtype_code(dtype), host_ptr(out), n, features))
    return out


def read_idx_labels(path, dtype=np.float64, classes=10) -> np.ndarray:
    (n,) = idx_shape(path)
    out = np.empty((n, classes), dtype=dtype)
    check(lib.sbb_read_idx_labels(os.fsencode(path), dtype_code(dtype), host_ptr(out), n, classes))
    return out


def load_mnist(image_file, label_file, dtype=np.float64):
    """train.py:9-23."""
    return read_idx_images(image_file, dtype), read_idx_labels(label_file, dtype, 10)


def _file_bytes(path) -> int:
    n = ctypes.c_long(0)
    check(lib.sbb_raw_u8_count(os.fsencode(path), ctypes.byref(n)))
    return int(n.value)


def load_stl_10_images(file, dtype=np.float64, features=STL10_FEATURES) -> np.ndarray:
    """train.py:26-31 (the reference always returns float64)."""
    size = _file_bytes(file)
    if size % features:
        raise ValueError("%s: %d bytes is not a whole number of %d-byte images" % (file, size, features))
    out = np.empty((size // features, features), dtype=dtype)
    check(lib.sbb_read_raw_u8_images(os.fsencode(file), dtype_code(dtype), host_ptr(out), out.shape[0], features))
    return out


def load_stl_10_labels(file, dtype=np.float64, classes=10) -> np.ndarray:
    """train.py:34-41: labels are stored 1-based."""
    n = _file_bytes(file)
    out = np.empty((n, classes), dtype=dtype)
    check(lib.sbb_read_raw_u8_labels(os.fsencode(file), dtype_code(dtype), host_ptr(out), n, classes, 1))
    return out
