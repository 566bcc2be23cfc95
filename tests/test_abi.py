"""The C-ABI library loads, exports every symbol the header declares, and refuses
to compute without a CUDA device.  No GPU needed."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import REPO


def _declared_symbols():
    text = open(os.path.join(REPO, "include", "sbb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sbb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from streambrain_b200 import _lib
    declared = _declared_symbols()
    assert len(declared) >= 30
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), "libsbb200.so does not export %s" % name
        assert name in _lib.SIGNATURES, "no ctypes signature for %s" % name
    assert sorted(_lib.SIGNATURES) == declared


def test_version_and_error_string():
    from streambrain_b200 import _lib
    assert _lib.lib.sbb_version() >= 100
    assert isinstance(_lib.lib.sbb_last_error(), bytes)


def test_invalid_arguments_are_rejected_before_any_device_work():
    from streambrain_b200 import _lib
    a = np.zeros((2, 4), dtype=np.float32)
    rc = _lib.lib.sbb_softmax_minicolumns(7, _lib.host_ptr(a), 2, 2, 2)
    assert rc == 1 and b"dtype" in _lib.lib.sbb_last_error()
    rc = _lib.lib.sbb_softmax_minicolumns(0, None, 2, 2, 2)
    assert rc == 1
    rc = _lib.lib.sbb_apply_mask(0, _lib.host_ptr(a), _lib.host_ptr(np.zeros((2, 2), dtype=np.uint8)), 2, 4, 2, 3)
    assert rc == 1 and b"shape" in _lib.lib.sbb_last_error()
    desc = _lib.LayerDesc(0, 5, 4, 2, 2, 0.01, 0, 0, 0, 16)
    h = ctypes.c_void_p()
    assert _lib.lib.sbb_layer_create(ctypes.byref(desc), ctypes.byref(h)) == 1
    assert not h.value


def test_wrapper_rejects_silent_conversions():
    from streambrain_b200 import kernels_b200 as k
    a64 = np.zeros((2, 4))
    with pytest.raises(TypeError):
        k.add_bias(a64, np.zeros(4, dtype=np.float32))
    with pytest.raises(TypeError):
        k.softmax_minicolumns(np.zeros((4, 4), dtype=np.float32)[:, ::2], 1, 2)
    with pytest.raises(Exception, match="Invalid dtype"):
        k.softmax_minicolumns(np.zeros((2, 4), dtype=np.int32), 2, 2)


def test_process_wide_settings_round_trip():
    """Settings that have no counterpart in the reference: host-side state only, so they work without a GPU."""
    from streambrain_b200._lib import check, lib
    before = lib.sbb_get_reserved_sms()
    try:
        check(lib.sbb_set_reserved_sms(24))
        assert lib.sbb_get_reserved_sms() == 24
        assert lib.sbb_set_reserved_sms(-1) != 0          # rejected, value kept
        assert lib.sbb_get_reserved_sms() == 24
    finally:
        check(lib.sbb_set_reserved_sms(before))
    path = lib.sbb_get_contraction_path()
    try:
        check(lib.sbb_set_contraction_path(0))
        assert lib.sbb_get_contraction_path() == 0
        assert lib.sbb_set_contraction_path(7) != 0
    finally:
        check(lib.sbb_set_contraction_path(path))


def test_no_cpu_fallback_without_a_device():
    from streambrain_b200 import _lib
    if _lib.lib.sbb_device_count() > 0:
        pytest.skip("a CUDA device is present")
    from streambrain_b200 import kernels_b200 as k
    with pytest.raises(_lib.SbbError) as e:
        k.softmax_minicolumns(np.zeros((2, 4), dtype=np.float32), 2, 2)
    assert e.value.code == 3
    import streambrain_b200 as B
    with pytest.raises(_lib.SbbError):
        B.DenseLayer(8, 1, 4, 0.01, (0.1, 0.1, 0.01), np.float32)
    # the allocation-free mask update follows the same contract (pointers are never touched without a device)
    fake = ctypes.c_void_p(256)
    rc = _lib.lib.sbb_update_mask_noalloc(0, fake, fake, fake, fake, fake, 0.01, 8, 4, 2, 2, 0, 1, None)
    assert rc == 3
    assert b"no CUDA device" in _lib.lib.sbb_noalloc_last_error()
    assert b"no CUDA device" in _lib.lib.sbb_last_error()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(REPO, "streambrain_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(root, f)).read()
                assert "oracle" not in src.lower() or f == "synthetic.py" and False, os.path.join(root, f)


def test_header_constants_match_the_binding():
    """The numeric constants the ctypes binding repeats (error codes, dtypes, layer kinds, state indices, the
    size of the sharding hand-shake) are the header's."""
    import re
    from conftest import REPO
    from streambrain_b200 import _lib
    text = open(os.path.join(REPO, "include", "sbb200.h")).read()
    defs = {m.group(1): int(m.group(2)) for m in re.finditer(r"^#define\s+(SBB_[A-Z0-9_]+)\s+(-?\d+)\b", text, re.M)}
    assert defs["SBB_OK"] == _lib.SBB_OK == 0
    for name, value in _lib.ERR_NAMES.items():
        assert defs[value] == name
    assert (defs["SBB_ERR_INVALID"], defs["SBB_ERR_CUDA"], defs["SBB_ERR_NO_DEVICE"], defs["SBB_ERR_UNSUPPORTED"],
            defs["SBB_ERR_TIMEOUT"]) == (_lib.ERR_INVALID, _lib.ERR_CUDA, _lib.ERR_NO_DEVICE, _lib.ERR_UNSUPPORTED,
                                         _lib.ERR_TIMEOUT)
    assert (defs["SBB_F32"], defs["SBB_F64"]) == (_lib.F32, _lib.F64)
    assert (defs["SBB_LAYER_DENSE"], defs["SBB_LAYER_PLASTIC"]) == (_lib.DENSE, _lib.PLASTIC)
    assert (defs["SBB_SHARD_BUFFERS"], defs["SBB_SHARD_HANDLE_BYTES"]) == (_lib.SHARD_BUFFERS, _lib.SHARD_HANDLE_BYTES)
    for name, index in _lib.STATE.items():
        key = {"weights": "WEIGHTS", "bias": "BIAS", "Ci": "CI", "Cj": "CJ", "Cij": "CIJ", "kbi": "KBI", "wmask": "WMASK"}[name]
        assert defs["SBB_STATE_" + key] == index
