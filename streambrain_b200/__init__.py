"""streambrain_b200 -- a B200-native backend for StreamBrain's BCPNN layers.

Importing this package plays the role of the reference's ``BCPNN`` package
(BCPNN/__init__.py:8-41): the environment variable ``BCPNN_BACKEND`` selects the
backend whose ``Network``, ``DenseLayer`` and ``StructuralPlasticityLayer`` are
re-exported, and ``backend()`` returns its name.  The value this package adds is
``b200`` (also the default here).  Any other value (``numpy``, ``cpu``, ``mpi``,
``gpu``, ``full_cuda``) belongs to the reference package and is forwarded to it
when a StreamBrain checkout is importable; otherwise the import fails with the
reference's own error message.

The backend is resolved lazily, on first attribute access, so that helper
modules (``streambrain_b200.synthetic``, ``streambrain_b200.build``) can be
imported before the shared library has been built.
"""
from __future__ import annotations

import importlib
import os
import sys

_EXPORTS = ("Network", "DenseLayer", "StructuralPlasticityLayer")
_BACKEND = os.environ.get("BCPNN_BACKEND", "b200")
_module = None


def backend():
    return _BACKEND


def _resolve():
    global _module
    if _module is not None:
        return _module
    if _BACKEND == "b200":
        sys.stderr.write("Using B200 backend.\n")
        _module = importlib.import_module(".backend.b200_backend", __name__)
    elif _BACKEND in ("numpy", "cpu", "mpi", "gpu", "full_cuda", "fpga"):
        try:
            _module = importlib.import_module("BCPNN")
        except ImportError as e:
            raise ValueError("Unable to import backend : %s (it belongs to the StreamBrain package, "
                             "which is not importable here: %s)" % (_BACKEND, e))
    else:
        raise ValueError("Unable to import backend : " + str(_BACKEND))
    return _module


def __getattr__(name):
    if name in _EXPORTS:
        return getattr(_resolve(), name)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))


def __dir__():
    return sorted(list(globals()) + list(_EXPORTS))
