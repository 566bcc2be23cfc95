"""The data-parallel train step over NCCL on two GPUs of one node: each rank runs
the pipelined step (row blocks of the batch outer product all-reduced while the
next block is computed) on its half of the batch; the replicas must stay
bit-identical and equal, within float32 summation-order tolerance, a single
GPU's step on the whole batch -- the equivalence the reference asserts for its
MPI backend (BCPNN/backend/_kernels/test_mpi.py:48-59).  Skipped with fewer than
two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from conftest import REPO, TOL, rel_inf, weight_err

pytestmark = pytest.mark.gpu

N, H, MC, B_LOCAL, TAU = 512, 8, 32, 96, 0.02
M = H * MC


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _make_layer(B200, path):
    from streambrain_b200._lib import check, lib
    check(lib.sbb_set_contraction_path(1 if path == "tensor" else 0))
    np.random.seed(11)
    layer = B200.StructuralPlasticityLayer(N, H, MC, TAU, -100.0, 0.05, 0.01, 0.5, 16, (1.0, 1.0 / MC, 1.0 / MC),
                                           dtype=np.float32)
    rs = np.random.RandomState(5)
    layer.Ci = (0.2 + 0.6 * rs.rand(N)).astype(np.float32)
    layer.Cj = (0.2 + 0.6 * rs.rand(M)).astype(np.float32) / MC
    # near independence: small weights keep the softmax of the second step well conditioned, so
    # that the two arithmetic orders (fused step / reduced sums) stay within the float32 tolerance
    layer.Cij = (np.outer(layer.Ci, layer.Cj) * (0.95 + 0.1 * rs.rand(N, M))).astype(np.float32)
    return layer


def _batches(world, steps):
    rs = np.random.RandomState(7)
    return [rs.rand(world * B_LOCAL, N).astype(np.float32) for _ in range(steps)]


def _worker(rank, world, port, path, out_dir, sharded=False, staged=False):
    sys.path.insert(0, REPO)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if os.environ.get("SBB_TEST_NVLS", "0") != "1":   # SBB_TEST_NVLS=1 leaves NCCL's NVLink-switch reductions on
        os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import streambrain_b200 as B200
    from streambrain_b200 import parallel
    layer = _make_layer(B200, path)
    if sharded:
        layer.shard_rows(rank, world, parallel.all_gather_bytes_over(dist), B_LOCAL)
        assert [layer.owned_rows(r) for r in range(world)] == parallel.shard_bounds(N, world)
    steps = 2
    all_reduce = lambda t: dist.all_reduce(t, async_op=True)
    batches = _batches(world, steps)
    mine = [torch.from_numpy(xb[rank * B_LOCAL:(rank + 1) * B_LOCAL]).cuda() for xb in batches]
    for k, xb in enumerate(batches):
        x = mine[k]
        if sharded:   # forward + train in one; a rank holds only its own rows until they are shared
            ahead = staged and k + 1 < steps   # the next batch's exchange runs beside this step
            layer.sharded_step(x, (2 + k) % H, all_reduce, next_inputs=mine[k + 1] if ahead else None)
            layer.share_rows(all_reduce)
        else:
            y = layer.compute_activation(x)
            layer.dp_train_step(x, y, (2 + k) % H, world, all_reduce, row_blocks=3)
        torch.cuda.synchronize()
        np.savez(os.path.join(out_dir, "rank%d_step%d.npz" % (rank, k)), Ci=layer.Ci, Cj=layer.Cj, Cij=layer.Cij,
                 weights=layer.weights, bias=layer.bias, wmask=layer.wmask)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("staged", [False, True])
@pytest.mark.parametrize("path", ["general", "tensor"])
def test_two_gpu_row_sharded_step_equals_allreduce_step(tmp_path, path, staged):
    """The row-sharded step (every rank owns half of the input rows: the ranks exchange the matching columns of
    their batches over NVLink, sum their parts of the supports, and each updates its own rows from the whole
    global batch) against the all-reduce step on the same two GPUs: the same traces, weights and masks to
    summation-order rounding."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    a, b = tmp_path / "allreduce", tmp_path / "sharded"
    a.mkdir()
    b.mkdir()
    mp.spawn(_worker, args=(world, _free_port(), path, str(a), False), nprocs=world, join=True)
    mp.spawn(_worker, args=(world, _free_port(), path, str(b), True, staged), nprocs=world, join=True)
    tol = TOL[np.dtype(np.float32)]
    for k in range(2):
        s0 = np.load(b / ("rank0_step%d.npz" % k))
        s1 = np.load(b / ("rank1_step%d.npz" % k))
        ref = np.load(a / ("rank0_step%d.npz" % k))
        for name in s0.files:
            assert np.array_equal(s0[name], s1[name]), (k, name)      # replicas identical
        assert np.array_equal(s0["wmask"], ref["wmask"]), k
        scale = 10 ** k
        for name in ("Ci", "Cj", "Cij", "bias"):
            assert rel_inf(s0[name], ref[name]) < scale * tol, (k, name)
        assert weight_err(s0["weights"], ref["weights"]) < 10 * scale * tol, k
        assert np.array_equal(s0["weights"] == 0, ref["weights"] == 0), k


@pytest.mark.parametrize("path", ["general", "tensor"])
def test_two_gpu_step_equals_big_batch(tmp_path, path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), path, str(tmp_path)), nprocs=world, join=True)
    got = []
    for k in range(2):
        r0 = np.load(tmp_path / ("rank0_step%d.npz" % k))
        r1 = np.load(tmp_path / ("rank1_step%d.npz" % k))
        for name in r0.files:
            assert np.array_equal(r0[name], r1[name]), name   # replicas stay identical
        got.append(r0)

    import streambrain_b200 as B200
    torch.cuda.set_device(0)

    class Done:
        def wait(self):
            pass

    # (a) the same kernels on one GPU with the whole batch (world_size 1, nothing to reduce): only the
    # order of the batch summation differs; (b) the fused single-device step, whose trace arithmetic is
    # ordered differently (kernels_openmp_internal.cc:361-383 against kernels_mpi_internal.cc:100-250).
    # One step is compared at the float32 tolerance.  The second step's forward pass amplifies the
    # first step's rounding differences in the weights (sums over all inputs, then a softmax), for
    # the summation orders of two ranks and of one alike, so it is compared ten times looser.
    whole, fused = _make_layer(B200, path), _make_layer(B200, path)
    tol = TOL[np.dtype(np.float32)]
    for k, xb in enumerate(_batches(world, 2)):
        for layer, scale in ((whole, 1), (fused, 10)):
            halves = [xb[r * B_LOCAL:(r + 1) * B_LOCAL] for r in range(world)]
            y = np.concatenate([layer.compute_activation(h) for h in halves])   # per-rank forward, as the workers do
            if layer is whole:
                layer.dp_train_step(torch.from_numpy(xb).cuda(), torch.from_numpy(y).cuda(), (2 + k) % H, 1,
                                    lambda t: Done(), row_blocks=3)
            else:
                layer.train_step(xb, y, (2 + k) % H)
            torch.cuda.synchronize()
            scale *= 10 ** k
            errs = {name: rel_inf(got[k][name], getattr(layer, name)) for name in ("Ci", "Cj", "Cij", "bias")}
            errs["weights"] = weight_err(got[k]["weights"], layer.weights)
            errs["wmask bits that differ"] = int((got[k]["wmask"] != layer.wmask).sum())
            assert errs["wmask bits that differ"] == 0, (k, errs)
            assert all(errs[name] < scale * tol for name in ("Ci", "Cj", "Cij", "bias")), (k, errs)
            assert errs["weights"] < 10 * scale * tol, (k, errs)


def _net_worker(rank, world, port, out_dir, sharded):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import streambrain_b200 as B200
    from streambrain_b200 import parallel
    from conftest import load_golden
    g = load_golden("network_f64.npz")
    net, x, lab, B, n_train = _golden_net(B200, g)

    def sum_counts(a):
        t = torch.from_numpy(np.asarray(a).copy()).cuda()
        dist.all_reduce(t)
        return t.cpu().numpy()

    net.set_data_parallel(rank, world, all_reduce=lambda t: dist.all_reduce(t, async_op=True), sum_counts=sum_counts,
                          all_gather_bytes=parallel.all_gather_bytes_over(dist) if sharded else None)
    net.fit(x[:n_train], lab[:n_train], B, [(0, 3)])
    net.fit(x[:n_train], lab[:n_train], B, [(1, 2)])
    correct, total = net.evaluate(x[n_train:], lab[n_train:], B)
    if sharded:   # the hidden layer was sharded by fit, which shares its rows at the end of every epoch
        assert net._layers[0]._shard == (rank, world) and getattr(net._layers[1], "_shard", None) is None
    torch.cuda.synchronize()
    out = {"correct": correct, "total": total, "wmask": net._layers[0].wmask}
    for li, layer in enumerate(net._layers):
        for name in ("Ci", "Cj", "Cij", "weights", "bias"):
            out["l%d_%s" % (li, name)] = getattr(layer, name)
    np.savez(os.path.join(out_dir, "net_rank%d.npz" % rank), **out)
    dist.barrier()
    dist.destroy_process_group()


def _golden_net(B200, g):
    import random
    n_pix, H, Mc, B = int(g["n_pix"]), int(g["H"]), int(g["Mc"]), int(g["B"])
    B -= B % 2                                     # two ranks halve every batch: keep them even
    n_train = int(g["n_train"])
    n_train -= n_train % 2
    np.random.seed(int(g["seed"]))
    random.seed(int(g["seed"]))
    net = B200.Network(np.float64)
    net.verbose = False
    net.add_layer(B200.StructuralPlasticityLayer(2 * n_pix, H, Mc, 0.03, -40.0, 0.1, 0.05, 0.5, 16,
                                                 (1, 1 / Mc, 1 / Mc)))
    net.add_layer(B200.DenseLayer(H * Mc, 1, 10, 0.02, (1 / Mc, 1 / 10, 1 / Mc / 10)))
    return net, g["x"], g["labels"], B, n_train


@pytest.mark.parametrize("sharded", [False, True])
def test_two_gpu_network_fit_equals_single_gpu_fit(tmp_path, sharded):
    """Network.fit / evaluate through the native loop on two ranks (each takes half of every batch, the trained
    layer sums its batch deltas over the ranks) against the same seeded run on one GPU: float64, so the
    masks must be identical and the state equal to summation-order rounding."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from conftest import load_golden
    world = 2
    mp.spawn(_net_worker, args=(world, _free_port(), str(tmp_path), sharded), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "net_rank0.npz"), np.load(tmp_path / "net_rank1.npz")
    for name in r0.files:
        assert np.array_equal(r0[name], r1[name]), name
    import streambrain_b200 as B200
    torch.cuda.set_device(0)
    g = load_golden("network_f64.npz")
    net, x, lab, B, n_train = _golden_net(B200, g)
    net.fit(x[:n_train], lab[:n_train], B, [(0, 3)])
    net.fit(x[:n_train], lab[:n_train], B, [(1, 2)])
    correct, total = net.evaluate(x[n_train:], lab[n_train:], B)
    assert np.array_equal(r0["wmask"], net._layers[0].wmask)
    for li, layer in enumerate(net._layers):
        for name in ("Ci", "Cj", "Cij", "bias", "weights"):
            assert rel_inf(r0["l%d_%s" % (li, name)], getattr(layer, name)) < 1e-9, (li, name)
    # every rank evaluates floor(batch / 2) samples of each batch (an odd last batch drops one sample)
    n_test = x.shape[0] - n_train
    expect_total = sum(2 * (min(B, n_test - s) // 2) for s in range(0, n_test, B))
    assert int(r0["total"][0]) == expect_total
    if expect_total == int(total[0]):
        assert int(r0["correct"][0]) == int(correct[0])
