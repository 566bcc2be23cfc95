"""Layer- and network-level parity on the GPU through the reference-facing API
(streambrain_b200.{StructuralPlasticityLayer, DenseLayer, Network}), against the
golden trajectories of the reference cpu backend and against the CPU oracle at
the MNIST-shaped configuration; full-size STL-10-shaped checks use properties that
do not need a full CPU run."""
import ctypes
import random

import numpy as np
import pytest

from conftest import TOL, load_golden, mask_mismatch_is_a_tie, rel_inf, weight_err

import oracle

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("contraction_path")]

DTYPES = [("f32", np.float32), ("f64", np.float64)]
PLASTIC_STATE = ("weights", "bias", "Ci", "Cj", "Cij", "kbi", "wmask")


@pytest.fixture(scope="module")
def B200():
    import streambrain_b200
    return streambrain_b200


def _layers_from_golden(B200, g, dtype):
    H, Mc, n_pix = int(g["H"]), int(g["Mc"]), int(g["n_pix"])
    np.random.seed(0)
    layer = B200.StructuralPlasticityLayer(2 * n_pix, H, Mc, float(g["hp_taupdt"]), float(g["hp_khalf"]),
                                           float(g["hp_pmin"]), float(g["hp_taubdt"]), float(g["hp_density"]), 16,
                                           (1, 1 / Mc, 1 / Mc), dtype=dtype)
    dense = B200.DenseLayer(H * Mc, 1, 10, float(g["dense_taupdt"]), (1 / Mc, 1 / 10, 1 / Mc / 10), dtype=dtype)
    for name in PLASTIC_STATE:
        setattr(layer, name, g["init_" + name])
    for name in ("weights", "bias", "Ci", "Cj", "Cij"):
        setattr(dense, name, g["dinit_" + name])
    return layer, dense


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_layer_steps_teacher_forced_vs_golden(B200, tag, dtype):
    g = load_golden("layer_%s.npz" % tag)
    tol = TOL[np.dtype(dtype)]
    layer, dense = _layers_from_golden(B200, g, dtype)
    B, steps, Mc = int(g["B"]), int(g["steps"]), int(g["Mc"])
    for s in range(steps):
        x = g["x"][s * B:(s + 1) * B]
        lab = g["labels"][s * B:(s + 1) * B]
        act = layer.compute_activation(x)
        assert rel_inf(act, g["act_%d" % s]) < tol, s
        assert rel_inf(dense.compute_activation(g["act_%d" % s]), g["dact_%d" % s]) < tol, s
        h = int(g["hs"][s])
        before = layer.wmask
        dense.train_step(g["act_%d" % s], lab)
        layer.train_step(x, g["act_%d" % s], None if h < 0 else h)
        for name in ("Ci", "Cj", "Cij", "kbi", "bias"):
            assert rel_inf(getattr(layer, name), g["s%d_%s" % (s, name)]) < tol, (s, name)
        got_mask = layer.wmask
        want = {n: g["s%d_%s" % (s, n)] for n in PLASTIC_STATE}
        if dtype == np.float64:
            assert np.array_equal(got_mask, want["wmask"]), s
        else:
            assert mask_mismatch_is_a_tie(got_mask, want["wmask"], max(h, 0), before, want,
                                          float(g["hp_taupdt"]) / 2, Mc, 1e-5), s
        if np.array_equal(got_mask, want["wmask"]):
            W = layer.weights
            assert weight_err(W, want["weights"]) < 10 * tol, s
            assert np.array_equal(W == 0, want["weights"] == 0), s
        for name in ("Ci", "Cj", "Cij"):
            assert rel_inf(getattr(dense, name), g["d%d_%s" % (s, name)]) < tol, (s, name)
        assert weight_err(dense.weights, g["d%d_weights" % s]) < 10 * tol, s
        for name in PLASTIC_STATE:
            setattr(layer, name, want[name])
        for name in ("weights", "Ci", "Cj", "Cij"):
            setattr(dense, name, g["d%d_%s" % (s, name)])
    dense.train_finalize()
    assert rel_inf(dense.bias, g["dfinal_bias"]) < tol


def test_layer_free_run_f64_vs_golden(B200):
    g = load_golden("layer_f64.npz")
    layer, _ = _layers_from_golden(B200, g, np.float64)
    B, steps = int(g["B"]), int(g["steps"])
    for s in range(steps):
        x = g["x"][s * B:(s + 1) * B]
        act = layer.compute_activation(x)
        h = int(g["hs"][s])
        layer.train_step(x, act, None if h < 0 else h)
        assert np.array_equal(layer.wmask, g["s%d_wmask" % s]), s
    assert rel_inf(layer.Cij, g["s%d_Cij" % (steps - 1)]) < 1e-10
    assert rel_inf(layer.weights, g["s%d_weights" % (steps - 1)]) < 1e-9


def test_device_tensor_path_equals_host_path(B200):
    """CUDA tensors in -> CUDA tensors out must give the same numbers as numpy in/out,
    and the fused host step (one upload) the same as forward + train_step."""
    import torch
    g = load_golden("layer_f32.npz")
    B = int(g["B"])
    x = g["x"][:B]
    la, _ = _layers_from_golden(B200, g, np.float32)
    lb, _ = _layers_from_golden(B200, g, np.float32)
    lc, _ = _layers_from_golden(B200, g, np.float32)
    ya = la.compute_activation(x)
    la.train_step(x, ya, 1)
    xt = torch.from_numpy(x).cuda()
    yb = lb.compute_activation(xt)
    lb.train_step(xt, yb, 1)
    torch.cuda.synchronize()
    yc = lc.step_host(x, None, 1)
    assert np.array_equal(ya, yb.cpu().numpy()) and np.array_equal(ya, yc)
    for name in PLASTIC_STATE:
        assert np.array_equal(getattr(la, name), getattr(lb, name)), name
        assert np.array_equal(getattr(la, name), getattr(lc, name)), name
    t = lb.state_tensor("Cij")
    assert t.is_cuda and np.array_equal(t.cpu().numpy(), lb.Cij)


def test_row_block_products_with_reserved_sms(B200):
    """The persistent row-block product may leave multiprocessors to a collective running beside
    it (sbb_set_reserved_sms): a smaller grid walks the same tiles and must give the same sums."""
    import torch
    from streambrain_b200._lib import check, lib

    class Done:
        def wait(self):
            pass

    g = load_golden("layer_f32.npz")
    B = int(g["B"])
    x = torch.from_numpy(np.ascontiguousarray(g["x"][:B])).cuda()
    full, _ = _layers_from_golden(B200, g, np.float32)
    fewer, _ = _layers_from_golden(B200, g, np.float32)
    y = full.compute_activation(x)
    full.dp_train_step(x, y, 1, 1, lambda t: Done(), row_blocks=2)
    try:
        check(lib.sbb_set_reserved_sms(140))
        fewer.dp_train_step(x, y, 1, 1, lambda t: Done(), row_blocks=2)
    finally:
        check(lib.sbb_set_reserved_sms(0))
    torch.cuda.synchronize()
    for name in PLASTIC_STATE:
        assert np.array_equal(getattr(fewer, name), getattr(full, name)), name


def test_async_host_steps_equal_blocking_host_steps(B200):
    """Five pipelined host-buffer steps (copies double-buffered against the steps, page-locked
    buffers) leave the same state and return the same activations as five blocking calls."""
    import torch
    g = load_golden("layer_f32.npz")
    B, steps = int(g["B"]), 5
    blocking, _ = _layers_from_golden(B200, g, np.float32)
    piped, _ = _layers_from_golden(B200, g, np.float32)
    xs = [torch.from_numpy(np.ascontiguousarray(g["x"][s * B:(s + 1) * B])).pin_memory() for s in range(steps)]
    outs = [torch.empty((B, piped.out_features), dtype=torch.float32).pin_memory() for _ in range(steps)]
    want = [blocking.step_host(xs[s].numpy(), None, s % 3) for s in range(steps)]
    for s in range(steps):
        piped.step_host_async(xs[s].numpy(), None, s % 3, out=outs[s].numpy())
    piped.wait()
    for s in range(steps):
        assert np.array_equal(outs[s].numpy(), want[s]), s
    for name in PLASTIC_STATE:
        assert np.array_equal(getattr(piped, name), getattr(blocking, name)), name
    # the blocking entry points work again after wait()
    assert np.array_equal(piped.step_host(xs[0].numpy(), None, 1), blocking.step_host(xs[0].numpy(), None, 1))


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_network_fit_and_evaluate_vs_golden(B200, tag, dtype):
    g = load_golden("network_%s.npz" % tag)
    n_pix, H, Mc, B = int(g["n_pix"]), int(g["H"]), int(g["Mc"]), int(g["B"])
    n_train, seed = int(g["n_train"]), int(g["seed"])
    np.random.seed(seed)
    random.seed(seed)
    net = B200.Network(dtype)
    net.verbose = False
    net.add_layer(B200.StructuralPlasticityLayer(2 * n_pix, H, Mc, 0.03, -40.0, 0.1, 0.05, 0.5, 16,
                                                 (1, 1 / Mc, 1 / Mc)))
    net.add_layer(B200.DenseLayer(H * Mc, 1, 10, 0.02, (1 / Mc, 1 / 10, 1 / Mc / 10)))
    x, lab = g["x"], g["labels"]
    net.fit(x[:n_train], lab[:n_train], B, [(0, 3)])
    net.fit(x[:n_train], lab[:n_train], B, [(1, 2)])
    correct, total = net.evaluate(x[n_train:], lab[n_train:], B)
    assert int(total[0]) == int(g["total"][0])
    if dtype == np.float64:
        assert np.array_equal(net._layers[0].wmask, g["l0_wmask"])
        for li, layer in enumerate(net._layers):
            for name in ("Ci", "Cj", "Cij", "bias", "weights"):
                assert rel_inf(getattr(layer, name), g["l%d_%s" % (li, name)]) < 1e-9, (li, name)
        assert int(correct[0]) == int(g["correct"][0])
        act = x[n_train:]
        for layer in net._layers:
            act = layer.compute_activation(act)
        assert np.array_equal(np.argmax(act, axis=1), g["test_pred"])
    else:
        for name in ("Ci", "Cj"):
            assert rel_inf(getattr(net._layers[0], name), g["l0_" + name]) < 1e-3, name


def _small_network(B200, g, dtype):
    n_pix, H, Mc = int(g["n_pix"]), int(g["H"]), int(g["Mc"])
    net = B200.Network(dtype)
    net.verbose = False
    net.add_layer(B200.StructuralPlasticityLayer(2 * n_pix, H, Mc, 0.03, -40.0, 0.1, 0.05, 0.5, 16,
                                                 (1, 1 / Mc, 1 / Mc)))
    net.add_layer(B200.DenseLayer(H * Mc, 1, 10, 0.02, (1 / Mc, 1 / 10, 1 / Mc / 10)))
    return net


def test_network_with_reduction_callbacks_reproduces_golden_run(B200):
    """The native loop with the data-parallel callbacks installed (one rank: the sum over ranks is the
    identity) runs the split step -- row-block products, reduction, row-block apply -- for every batch
    and must land on the reference's golden run like the fused step does."""
    g = load_golden("network_f64.npz")
    B, n_train, seed = int(g["B"]), int(g["n_train"]), int(g["seed"])
    np.random.seed(seed)
    random.seed(seed)
    net = _small_network(B200, g, np.float64)

    class Done:
        def wait(self):
            pass

    started = []
    net.set_data_parallel(0, 1, all_reduce=lambda t: started.append(t.numel()) or Done())
    x, lab = g["x"], g["labels"]
    net.fit(x[:n_train], lab[:n_train], B, [(0, 3)])
    net.fit(x[:n_train], lab[:n_train], B, [(1, 2)])
    correct, total = net.evaluate(x[n_train:], lab[n_train:], B)
    assert len(started) > 0
    assert np.array_equal(net._layers[0].wmask, g["l0_wmask"])
    for li, layer in enumerate(net._layers):
        for name in ("Ci", "Cj", "Cij", "bias", "weights"):
            assert rel_inf(getattr(layer, name), g["l%d_%s" % (li, name)]) < 1e-9, (li, name)
    assert int(correct[0]) == int(g["correct"][0]) and int(total[0]) == int(g["total"][0])


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_checkpoint_resume_equals_uninterrupted_run(B200, tmp_path, tag, dtype):
    """save() after two epochs, load() into a fresh network, continue: bit-identical to the run that was
    never interrupted (the random stream is carried over as well, as a resumed job would)."""
    g = load_golden("network_%s.npz" % tag)
    B, n_train = int(g["B"]), int(g["n_train"])
    x, lab = g["x"][:n_train], g["labels"][:n_train]

    np.random.seed(5)
    whole = _small_network(B200, g, dtype)
    whole.fit(x, lab, B, [(0, 2)])
    whole.fit(x, lab, B, [(0, 2), (1, 1)])

    np.random.seed(5)
    first = _small_network(B200, g, dtype)
    first.fit(x, lab, B, [(0, 2)])
    first.save(tmp_path / "ckpt.npz")
    rng = np.random.get_state()
    del first

    np.random.seed(99)                      # a fresh process: other initial weights, another stream
    resumed = _small_network(B200, g, dtype)
    resumed.load(tmp_path / "ckpt.npz")
    np.random.set_state(rng)
    resumed.fit(x, lab, B, [(0, 2), (1, 1)])
    for a, b in zip(whole._layers, resumed._layers):
        for name in a._state_names:
            assert np.array_equal(getattr(a, name), getattr(b, name)), name
    assert np.array_equal(whole.evaluate(g["x"][n_train:], g["labels"][n_train:], B)[0],
                          resumed.evaluate(g["x"][n_train:], g["labels"][n_train:], B)[0])
    with pytest.raises(ValueError):
        B200.Network(dtype).load(tmp_path / "ckpt.npz")     # layer count mismatch


def test_network_too_few_batches_for_the_mask_schedule(B200):
    np.random.seed(0)
    net = B200.Network(np.float32)
    net.verbose = False
    net.add_layer(B200.StructuralPlasticityLayer(8, 4, 2, 0.05, -10.0, 0.1, 0.1, 0.5, 16, (1, 0.5, 0.5)))
    net.add_layer(B200.DenseLayer(8, 1, 10, 0.05, (0.5, 0.1, 0.05)))
    from streambrain_b200 import synthetic
    x, lab = synthetic.make_inputs(16, 4, 0.5, np.float32)
    with pytest.raises(ZeroDivisionError):
        net.fit(x, lab, 8, [(0, 2)])
    net.fit(x, lab, 8, [(0, 1)])
    correct, total = net.evaluate(x, lab, 8)
    assert int(total[0]) == 16 and 0 <= int(correct[0]) <= 16


def _mnist_pair(B200, port_kernels, dtype, seed=0):
    from streambrain_b200 import synthetic
    p = synthetic.layer_params("mnist_f32" if dtype == np.float32 else "mnist_f64")
    hp = p["hidden"]
    np.random.seed(seed)
    dev = B200.StructuralPlasticityLayer(hp["in_features"], hp["hypercolumns"], hp["minicolumns"], hp["taupdt"],
                                         hp["khalf"], hp["pmin"], hp["taubdt"], hp["density"], 16,
                                         hp["initial_counters"], dtype=dtype)
    np.random.seed(seed)
    ref = oracle.OracleLayer(port_kernels, "plastic", hp["in_features"], hp["hypercolumns"], hp["minicolumns"],
                             hp["taupdt"], hp["initial_counters"], dtype, khalf=hp["khalf"], pmin=hp["pmin"],
                             taubdt=hp["taubdt"], density=hp["density"])
    x, lab = synthetic.make_inputs(p["batch"] * 6, p["n_pixels"], p["sparsity"], dtype)
    return dev, ref, x, lab, p


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_mnist_shaped_layer_teacher_forced_vs_oracle(B200, port_kernels, tag, dtype):
    """1568 -> 30x100, batch 128: identical seeded initial state (the constructor draws
    from the global NumPy stream in the reference's order), six steps, mask update from
    the third step on, every step restarted from the oracle's state."""
    dev, ref, x, _, p = _mnist_pair(B200, port_kernels, dtype)
    tol = TOL[np.dtype(dtype)]
    for name in PLASTIC_STATE:
        assert np.array_equal(getattr(dev, name), getattr(ref, name)), name
    B = p["batch"]
    Mc = p["hidden"]["minicolumns"]
    for s in range(6):
        xb = x[s * B:(s + 1) * B]
        a_ref = ref.compute_activation(xb)
        a_dev = dev.compute_activation(xb)
        assert rel_inf(a_dev, a_ref) < tol, s
        h = (7 * s) % 30 if s >= 2 else None
        before = ref.wmask.copy()
        ref.train_step(xb, a_ref, h)
        dev.train_step(xb, a_ref, h)
        for name in ("Ci", "Cj", "Cij", "kbi", "bias"):
            assert rel_inf(getattr(dev, name), getattr(ref, name)) < tol, (s, name)
        got = dev.wmask
        if dtype == np.float64:
            assert np.array_equal(got, ref.wmask), s
        else:
            assert mask_mismatch_is_a_tie(got, ref.wmask, h or 0, before, ref.state(), p["hidden"]["taupdt"] / 2, Mc,
                                          1e-5), s
        if np.array_equal(got, ref.wmask):
            assert weight_err(dev.weights, ref.weights) < 10 * tol, s
        for name in PLASTIC_STATE:
            setattr(dev, name, getattr(ref, name))


def test_mnist_shaped_argmax_predictions_identical(B200, port_kernels):
    """Classifier argmax on held-out samples after identical (teacher-forced) training state."""
    from streambrain_b200 import synthetic
    dev, ref, x, lab, p = _mnist_pair(B200, port_kernels, np.float64)
    op = p["out"]
    np.random.seed(1)
    dev_out = B200.DenseLayer(op["in_features"], 1, 10, op["taupdt"], op["initial_counters"], dtype=np.float64)
    np.random.seed(1)
    ref_out = oracle.OracleLayer(port_kernels, "dense", op["in_features"], 1, 10, op["taupdt"],
                                 op["initial_counters"], np.float64)
    B = p["batch"]
    for s in range(4):
        xb, lb = x[s * B:(s + 1) * B], lab[s * B:(s + 1) * B]
        a = ref.compute_activation(xb)
        ref_out.train_step(a, lb)
        dev_out.train_step(a, lb)
    ref_out.train_finalize()
    dev_out.train_finalize()
    xt = x[4 * B:]
    hidden = ref.compute_activation(xt)
    assert np.array_equal(np.argmax(dev_out.compute_activation(hidden), axis=1),
                          np.argmax(ref_out.compute_activation(hidden), axis=1))
    assert np.array_equal(np.argmax(dev_out.compute_activation(dev.compute_activation(xt)), axis=1),
                          np.argmax(ref_out.compute_activation(hidden), axis=1))


def test_data_parallel_split_step_equals_single_step(B200):
    """Two ranks emulated on one GPU through the C ABI: each half batch fills its own
    delta buffer, the buffers are summed (standing in for the allreduce), and the
    apply calls must reproduce the single-device step on the whole batch."""
    import torch
    from streambrain_b200._lib import check, lib
    g = load_golden("layer_f64.npz")
    B = int(g["B"])
    x = torch.from_numpy(g["x"][:B]).cuda()
    single, _ = _layers_from_golden(B200, g, np.float64)
    split, _ = _layers_from_golden(B200, g, np.float64)
    y = single.compute_activation(x)
    single.train_step(x, y, 2)
    n = int(lib.sbb_layer_delta_elems(split._handle))
    N = split.in_features
    deltas = [torch.zeros(n, dtype=torch.float64, device="cuda") for _ in range(2)]
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    half = B // 2
    for r in range(2):
        xs, ys = x[r * half:(r + 1) * half].contiguous(), y[r * half:(r + 1) * half].contiguous()
        check(lib.sbb_layer_dp_local(split._handle, xs.data_ptr(), ys.data_ptr(), half, deltas[r].data_ptr(), 0, N, st))
    total = deltas[0] + deltas[1]
    check(lib.sbb_layer_dp_apply_vectors(split._handle, total.data_ptr(), B, st))
    check(lib.sbb_layer_dp_apply_rows(split._handle, total.data_ptr(), B, 0, N, st))
    check(lib.sbb_layer_dp_finish(split._handle, 2, st))
    torch.cuda.synchronize()
    assert np.array_equal(split.wmask, single.wmask)
    for name in ("Ci", "Cj", "Cij", "weights", "bias", "kbi"):
        assert rel_inf(getattr(split, name), getattr(single, name)) < 1e-12, name
    # the pipelined orchestration with a local stand-in for the reduction (world_size 1)
    piped, _ = _layers_from_golden(B200, g, np.float64)

    class Done:
        def wait(self):
            pass

    piped.dp_train_step(x, y, 2, 1, lambda t: Done(), row_blocks=3)
    torch.cuda.synchronize()
    for name in ("Ci", "Cj", "Cij", "weights", "bias", "kbi", "wmask"):
        assert rel_inf(getattr(piped, name), getattr(single, name)) < 1e-12, name


@pytest.mark.parametrize("tag,dtype", DTYPES)
def test_row_sharded_step_on_one_rank_equals_single_step(B200, tag, dtype):
    """The row-sharded step with a world of one rank (it owns every row; the scatter, the partial forward
    product, the activation and the row-block update all run locally) must reproduce forward + fused step."""
    import torch
    g = load_golden("layer_%s.npz" % tag)
    B = int(g["B"])
    x = torch.from_numpy(np.ascontiguousarray(g["x"][:B])).cuda()
    single, _ = _layers_from_golden(B200, g, dtype)
    sharded, _ = _layers_from_golden(B200, g, dtype)
    sharded.shard_rows(0, 1, lambda blob: [blob], B)
    assert sharded.owned_rows() == (0, sharded.in_features)
    tol = TOL[np.dtype(dtype)]
    done = type("Done", (), {"wait": lambda self: None})
    for h in (2, None, 0):
        y = single.compute_activation(x)
        single.train_step(x, y, h)
        ys = sharded.sharded_step(x, h, lambda t: done())
        torch.cuda.synchronize()
        assert rel_inf(ys.cpu().numpy(), y.cpu().numpy() if hasattr(y, "cpu") else y) < tol, h
        assert np.array_equal(sharded.wmask, single.wmask), h
        for name in ("Ci", "Cj", "Cij", "bias", "kbi"):
            assert rel_inf(getattr(sharded, name), getattr(single, name)) < tol, (h, name)
        assert weight_err(sharded.weights, single.weights) < 10 * tol, h
        for name in PLASTIC_STATE:          # both continue from the same state
            setattr(sharded, name, getattr(single, name))
    # the same with every next batch staged ahead on the side stream (three input buffers used in turn)
    xs = [torch.from_numpy(np.ascontiguousarray(g["x"][:B] * s)).cuda() for s in (1.0, 0.5, 0.25, 0.75, 1.0)]
    for k, h in enumerate((1, None, 3, 0)):
        y = single.compute_activation(xs[k])
        single.train_step(xs[k], y, h)
        ys = sharded.sharded_step(xs[k], h, lambda t: done(), next_inputs=xs[k + 1])
        torch.cuda.synchronize()
        assert rel_inf(ys.cpu().numpy(), y.cpu().numpy() if hasattr(y, "cpu") else y) < tol * 10 ** k, k
        assert np.array_equal(sharded.wmask, single.wmask), k
        for name in ("Ci", "Cj", "Cij", "bias", "kbi"):
            assert rel_inf(getattr(sharded, name), getattr(single, name)) < tol * 10 ** k, (k, name)
    with pytest.raises(ValueError):         # the batch staged ahead must be the next one passed
        sharded.sharded_step(xs[0], None, lambda t: done())
    sharded.drop_staged()
    sharded.sharded_step(xs[0], None, lambda t: done())
    with pytest.raises(Exception):          # the plain data-parallel step refuses a sharded layer
        sharded.dp_train_step(x, y, None, 1, lambda t: done())
    big = torch.zeros((B + 1, sharded.in_features), dtype=x.dtype, device="cuda")
    with pytest.raises(Exception):          # more samples than the gathered-input buffers were sized for
        sharded.sharded_step(big, None, lambda t: done())


def test_stl10_shaped_layer_full_size_properties(B200, port_kernels):
    """55296 -> 30x100, batch 256, float32 (663 MB trace matrix).  Checked without a full
    CPU run: (a) the forward pass of a sample of batch rows against the oracle;
    (b) the trace update of a sample of input rows against the oracle (row i of Cij
    depends only on column i of x); (c) identities that hold for every row --
    sum_j Cij[i, HC] moves with Ci[i] because each hypercolumn's activations sum to
    one, and complementary input pairs satisfy Cij[2k] + Cij[2k+1] = Cj's update."""
    from streambrain_b200 import synthetic
    p = synthetic.layer_params("stl10_f32")
    hp = p["hidden"]
    N, H, Mc, B = hp["in_features"], hp["hypercolumns"], hp["minicolumns"], p["batch"]
    M = H * Mc
    np.random.seed(0)
    dev = B200.StructuralPlasticityLayer(N, H, Mc, hp["taupdt"], hp["khalf"], hp["pmin"], hp["taubdt"],
                                         hp["density"], 16, hp["initial_counters"], dtype=np.float32)
    x, _ = synthetic.make_inputs(B, p["n_pixels"], 0.0, np.float32)
    W0, b0, mask0 = dev.weights, dev.bias, dev.wmask
    y = dev.compute_activation(x)
    rows = [0, 1, 100, 255]
    s = port_kernels.update_state(np.zeros((len(rows), M), dtype=np.float32), W0, b0, np.ascontiguousarray(x[rows]))
    want = port_kernels.softmax_minicolumns(s, H, Mc)
    # K = 55296 float32 accumulations: the oracle's own rounding (sequential sums) is of the
    # order of 1e-4 here, so both are measured against a float64 evaluation of the same rows.
    s64 = x[rows].astype(np.float64) @ W0.astype(np.float64) + b0.astype(np.float64)
    y64 = oracle.numpy_softmax_minicolumns(s64, H, Mc)
    err_dev, err_ref = rel_inf(y[rows], y64), rel_inf(want, y64)
    assert err_dev < max(2 * err_ref, 1e-5), (err_dev, err_ref)
    assert rel_inf(y[rows], want) < 1e-3
    assert np.allclose(y.reshape(B, H, Mc).sum(axis=2), 1.0, atol=1e-5)

    Ci0, Cj0, Cij0 = dev.Ci, dev.Cj, dev.Cij
    dev.train_step(x, y, 3)
    Ci1, Cj1, Cij1, W1, mask1 = dev.Ci, dev.Cj, dev.Cij, dev.weights, dev.wmask
    pick = np.r_[0:8, 27640:27656, N - 8:N]
    sub = [Ci0[pick].copy(), Cj0.copy(), np.ascontiguousarray(Cij0[pick]), np.ascontiguousarray(x[:, pick]), y]
    taupdt = hp["taupdt"]
    cw = np.zeros((len(pick), M), dtype=np.float32)
    port_kernels.update_weights(sub[0], sub[1], sub[2], sub[3], sub[4], taupdt, cw, taupdt / 2)
    assert rel_inf(Ci1[pick], sub[0]) < 1e-5 and rel_inf(Cj1, sub[1]) < 1e-5
    assert rel_inf(Cij1[pick], sub[2]) < 1e-5
    masked = np.repeat(mask1[pick], Mc, axis=1).astype(bool)
    assert rel_inf(W1[pick], np.where(masked, cw, 0)) < 1e-4
    assert (W1[np.repeat(mask1, Mc, axis=1) == 0] == 0).all()   # silent connections carry no weight
    # (c) identities over ALL rows
    t = np.float64(np.float32(taupdt))
    row_sum = Cij1.astype(np.float64).reshape(N, H, Mc).sum(axis=2)
    expect = (1 - t) * Cij0.astype(np.float64).reshape(N, H, Mc).sum(axis=2) + \
        t * x.astype(np.float64).mean(axis=0)[:, None]
    assert np.abs(row_sum - expect).max() < 1e-5
    pair = Cij1[0::2].astype(np.float64) + Cij1[1::2].astype(np.float64)
    expect = (1 - t) * (Cij0[0::2].astype(np.float64) + Cij0[1::2]) + t * y.astype(np.float64).mean(axis=0)[None, :]
    assert np.abs(pair - expect).max() < 1e-6
    # mask update moved at most 16 connections in hypercolumn 3 and nothing else
    assert np.array_equal(np.delete(mask1, 3, axis=1), np.delete(mask0, 3, axis=1))
    assert mask1[:, 3].sum() == mask0[:, 3].sum() and (mask1[:, 3] != mask0[:, 3]).sum() <= 32


def test_errors_are_reported_not_fatal(B200):
    from streambrain_b200 import _lib
    np.random.seed(0)
    layer = B200.StructuralPlasticityLayer(8, 2, 2, 0.01, -10.0, 0.1, 0.1, 0.5, 16, (1, 0.5, 0.5), dtype=np.float32)
    with pytest.raises(ValueError):
        layer.compute_activation(np.zeros((4, 9), dtype=np.float32))
    with pytest.raises(ValueError):
        layer.weights = np.zeros((3, 3))
    with pytest.raises(_lib.SbbError) as e:
        layer.train_step(np.zeros((4, 8), dtype=np.float32), np.zeros((4, 4), dtype=np.float32), 5)
    assert e.value.code == 1
    rc = _lib.lib.sbb_layer_forward(layer._handle, None, 4, None, None)
    assert rc == 1
    buf = np.zeros(3, dtype=np.float32)
    assert _lib.lib.sbb_layer_get_state(layer._handle, 0, _lib.host_ptr(buf), buf.nbytes) == 1
    dense = B200.DenseLayer(8, 1, 4, 0.01, (0.5, 0.25, 0.125), dtype=np.float32)
    with pytest.raises(AttributeError):
        dense.kbi
    # the layer still works after the rejected calls
    out = layer.compute_activation(np.random.rand(4, 8).astype(np.float32))
    assert np.allclose(out.reshape(4, 2, 2).sum(axis=2), 1.0, atol=1e-6)
    assert _lib.lib.sbb_kernel_launches() > 0
