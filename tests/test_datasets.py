"""Dataset readers (IDX and STL-10 binaries) on files written by the test in those formats, and the
per-dataset hyper-parameter table.  Host code only: no GPU needed."""
import math
import struct

import numpy as np
import pytest


def _write_idx(path, array):
    array = np.ascontiguousarray(array, dtype=np.uint8)
    with open(path, "wb") as f:
        f.write(bytes([0, 0, 0x08, array.ndim]))
        for d in array.shape:
            f.write(struct.pack(">I", d))
        f.write(array.tobytes())


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_idx_files_read_like_the_reference_loader(tmp_path, dtype):
    from streambrain_b200 import datasets
    rs = np.random.RandomState(3)
    pixels = rs.randint(0, 256, size=(37, 28, 28)).astype(np.uint8)
    labels = rs.randint(0, 10, size=37).astype(np.uint8)
    _write_idx(tmp_path / "img", pixels)
    _write_idx(tmp_path / "lab", labels)
    assert datasets.idx_shape(tmp_path / "img") == (37, 28, 28)
    imgs, onehot = datasets.load_mnist(tmp_path / "img", tmp_path / "lab", dtype=dtype)
    # what train.py:9-23 computes: drop the 16 / 8 header bytes, reshape, scale, one-hot
    raw = np.fromfile(tmp_path / "img", dtype=np.uint8)[16:]
    want = np.reshape(raw, [-1, 28 * 28]).astype(dtype)
    want /= 255.0
    lraw = np.fromfile(tmp_path / "lab", dtype=np.uint8)[8:]
    want_l = np.zeros([lraw.shape[0], 10]).astype(dtype)
    want_l[np.arange(lraw.shape[0]), lraw] = 1.0
    assert imgs.dtype == dtype and np.array_equal(imgs, want)
    assert onehot.dtype == dtype and np.array_equal(onehot, want_l)


def test_stl10_binaries_read_like_the_reference_loader(tmp_path):
    from streambrain_b200 import datasets
    rs = np.random.RandomState(4)
    raw = rs.randint(0, 256, size=(5, 3 * 96 * 96)).astype(np.uint8)
    lab = rs.randint(1, 11, size=5).astype(np.uint8)
    raw.tofile(tmp_path / "X.bin")
    lab.tofile(tmp_path / "y.bin")
    x = datasets.load_stl_10_images(tmp_path / "X.bin")
    y = datasets.load_stl_10_labels(tmp_path / "y.bin")
    assert x.dtype == np.float64 and np.array_equal(x, raw / 255.0)      # train.py:26-31
    want = np.zeros([5, 10])
    want[np.arange(5), lab - 1] = 1.0                                       # train.py:34-41
    assert np.array_equal(y, want)
    assert np.array_equal(datasets.load_stl_10_images(tmp_path / "X.bin", np.float32), (raw / 255.0).astype(np.float32))


def test_malformed_files_raise(tmp_path):
    from streambrain_b200 import _lib, datasets
    with pytest.raises(_lib.SbbError, match="cannot open"):
        datasets.idx_shape(tmp_path / "missing")
    (tmp_path / "junk").write_bytes(b"\x01\x02\x03\x04" + bytes(100))
    with pytest.raises(_lib.SbbError, match="magic"):
        datasets.read_idx_images(tmp_path / "junk")
    _write_idx(tmp_path / "ok", np.zeros((4, 3, 3), dtype=np.uint8))
    data = (tmp_path / "ok").read_bytes()
    (tmp_path / "short").write_bytes(data[:-5])
    with pytest.raises(_lib.SbbError, match="bytes on disk"):
        datasets.read_idx_images(tmp_path / "short")
    (tmp_path / "int32").write_bytes(bytes([0, 0, 0x0C, 1]) + struct.pack(">I", 2) + bytes(8))
    with pytest.raises(_lib.SbbError, match="element type"):
        datasets.idx_shape(tmp_path / "int32")
    _write_idx(tmp_path / "badlab", np.array([1, 2, 11], dtype=np.uint8))
    with pytest.raises(_lib.SbbError, match="label"):
        datasets.read_idx_labels(tmp_path / "badlab")
    np.array([0, 3], dtype=np.uint8).tofile(tmp_path / "zero_based")
    with pytest.raises(_lib.SbbError, match="label"):
        datasets.load_stl_10_labels(tmp_path / "zero_based")       # STL-10 labels start at 1
    (tmp_path / "odd").write_bytes(bytes(100))
    with pytest.raises(ValueError):
        datasets.load_stl_10_images(tmp_path / "odd")


def test_hyperparameter_table_scales_with_the_batch_size():
    from streambrain_b200 import hyperparameters as hpm
    base = hpm.for_dataset("mnist", 128)
    big = hpm.for_dataset("mnist", 512)
    assert base["l1_taupdt"] == 0.006908854922437549 and base["l2_taupdt"] == 0.0007449780036161324
    assert big["l1_taupdt"] == base["l1_taupdt"] * math.sqrt(4) and big["l2_taupdt"] == base["l2_taupdt"] * 2
    assert (base["n_hypercolumns"], base["n_minicolumns"], base["n_hidden"]) == (15, 200, 3000)
    stl = hpm.for_dataset("stl-10", 128)
    assert stl["n_inputs"] == 27648 and stl["l1_mask_iterations"] == 584 and stl["l1_khalf"] > 0
    assert hpm.for_dataset("fashion_mnist", 128)["n_minicolumns"] == 100
    with pytest.raises(ValueError):
        hpm.for_dataset("cifar", 128)


@pytest.mark.gpu
def test_training_driver_runs_on_idx_files(tmp_path, monkeypatch, capsys):
    """The reference's driver (train.py:44-202) on this backend, on small IDX files written here: 200 training
    and 50 test images, two epochs of the hidden layer (the second one with mask updates) and one of the
    classifier."""
    from streambrain_b200 import hyperparameters, train
    rs = np.random.RandomState(0)
    for stem, n in (("train", 200), ("t10k", 50)):
        _write_idx(tmp_path / ("%s-images-idx3-ubyte" % stem), rs.randint(0, 256, size=(n, 28, 28)).astype(np.uint8))
        _write_idx(tmp_path / ("%s-labels-idx1-ubyte" % stem), rs.randint(0, 10, size=n).astype(np.uint8))
    short = dict(hyperparameters.DATASETS["mnist"], l1_epochs=2, l2_epochs=1)
    monkeypatch.setitem(hyperparameters.DATASETS, "mnist", short)
    from streambrain_b200.backend import b200_backend
    monkeypatch.setattr(b200_backend.Network, "verbose", False)
    assert train.main(["train", "mnist", "single", "8", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "Accuracy:" in out and "Training duration:" in out
