"""The data-parallel step on CPU: two gloo ranks run the pipelined orchestration
(streambrain_b200.parallel) with numpy arithmetic standing in for the CUDA ops,
and the result must equal the oracle's single-process step on the concatenated
batch -- the equivalence the reference asserts for its MPI backend
(BCPNN/backend/_kernels/test_mpi.py:48-59).  The network driver's batch slicing
under world_size 2 is checked the same way.  No GPU needed."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import REPO, rel_inf

N, H, MC, B_LOCAL, TAU = 300, 3, 4, 6, 0.05
M = H * MC


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class NumpyDPOps:
    """numpy implementation of the ops protocol (arithmetic of
    kernels_mpi_internal.cc:100-250 with the weight formula of the oracle)."""

    def __init__(self, state):
        self.s = state
        self.n_rows, self.n_cols = N, M
        self.delta = torch.zeros(N + M + N * M, dtype=torch.float64)
        self.calls = []

    def local(self, x, y, rb, re):
        d = self.delta.numpy()
        if rb == 0:
            d[:N] = x.sum(axis=0)
            d[N:N + M] = y.sum(axis=0)
        d[N + M + rb * M:N + M + re * M] = (x[:, rb:re].T @ y).ravel()
        self.calls.append(("local", rb, re))

    def _ema(self, old, s, batch):
        return np.maximum(0.0, old * (1.0 - TAU) + (s / batch) * TAU)

    def apply_vectors(self, batch):
        d = self.delta.numpy()
        self.s["Ci"] = self._ema(self.s["Ci"], d[:N], batch)
        self.s["Cj"] = self._ema(self.s["Cj"], d[N:N + M], batch)
        self.calls.append(("vectors",))

    def apply_rows(self, batch, rb, re):
        d = self.delta.numpy()[N + M + rb * M:N + M + re * M].reshape(re - rb, M)
        cthr = TAU / 2
        cij = self._ema(self.s["Cij"][rb:re], d, batch)
        self.s["Cij"][rb:re] = cij
        ci, cj = self.s["Ci"][rb:re, None], self.s["Cj"][None, :]
        w = np.log(np.maximum(cij, cthr ** 4) / (ci * cj))
        self.s["weights"][rb:re] = np.where((ci < cthr) | (cj < cthr), 0.0, w)
        self.calls.append(("rows", rb, re))

    def finish(self, h):
        self.calls.append(("finish", h))


def _dp_worker(rank, world, port, out_dir):
    sys.path.insert(0, REPO)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from streambrain_b200 import parallel
    rs = np.random.RandomState(0)
    state = dict(Ci=rs.rand(N), Cj=rs.rand(M), Cij=rs.rand(N, M), weights=np.zeros((N, M)))
    x = rs.rand(world * B_LOCAL, N)
    y = rs.rand(world * B_LOCAL, M)
    ops = NumpyDPOps(state)
    sl = slice(rank * B_LOCAL, (rank + 1) * B_LOCAL)
    parallel.pipelined_dp_step(ops, x[sl], y[sl], 2, B_LOCAL, world,
                               lambda t: dist.all_reduce(t, async_op=True), row_blocks=3)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), calls=np.array(repr(ops.calls)), **state)
    dist.destroy_process_group()


def test_two_rank_step_equals_big_batch(tmp_path, port_kernels):
    world = 2
    mp.spawn(_dp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0 = np.load(tmp_path / "rank0.npz")
    r1 = np.load(tmp_path / "rank1.npz")
    rs = np.random.RandomState(0)
    Ci, Cj, Cij = rs.rand(N), rs.rand(M), rs.rand(N, M)
    x = rs.rand(world * B_LOCAL, N)
    y = rs.rand(world * B_LOCAL, M)
    W = np.zeros((N, M))
    port_kernels.update_weights(Ci, Cj, Cij, x, y, TAU, W, TAU / 2)
    for name, want in (("Ci", Ci), ("Cj", Cj), ("Cij", Cij), ("weights", W)):
        assert np.array_equal(r0[name], r1[name]), name       # replicas stay identical
        assert rel_inf(r0[name], want) < 1e-12, name
    calls = eval(str(r0["calls"]))
    kinds = [c[0] for c in calls]
    assert kinds == ["local"] * 3 + ["vectors", "rows", "rows", "rows", "finish"]
    assert [c[1] for c in calls if c[0] == "local"] == [0, 128, 256]
    assert calls[-1] == ("finish", 2)


def _net_worker(rank, world, port, out_dir):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from streambrain_b200 import synthetic
    sys.path.insert(0, os.path.join(REPO, "tests"))
    from plan_driver import PlanNetwork

    seen = []

    class Recorder(oracle.OracleLayer):
        def train_step(self, inputs, outputs, hypercolumn=None):
            seen.append((inputs.shape[0], float(inputs[:, 0::2].sum()), hypercolumn))

    np.random.seed(3)
    net = PlanNetwork(np.float64, rank, world)
    net.add_layer(Recorder(oracle.PortKernels(), "plastic", 16, 2, 3, 0.05, (1, 1 / 3, 1 / 3), np.float64,
                           khalf=-10.0, pmin=0.1, taubdt=0.1, density=0.5))
    net.add_layer(Recorder(oracle.PortKernels(), "dense", 6, 1, 10, 0.05, (1 / 3, 0.1, 1 / 30), np.float64))
    x, lab = synthetic.make_inputs(35, 8, 0.5, np.float64)
    net.fit(x, lab, 10, [(0, 2)])
    correct, total = net.evaluate(x, lab, 10)
    correct, total = _sum(correct), _sum(total)   # the mpi backend's Allreduce of the counters
    np.savez(os.path.join(out_dir, "net%d.npz" % rank), seen=np.array(repr(seen)), total=total, correct=correct)
    dist.destroy_process_group()


def _sum(a):
    t = torch.from_numpy(np.asarray(a).copy())
    dist.all_reduce(t)
    return t.numpy()


def test_network_slices_batches_per_rank(tmp_path):
    """35 samples, batch 10, 2 ranks: each rank takes 5 of every full batch and 2 of
    the last partial one (5 // 2, the odd sample is dropped) --
    _cpu_base_backend.py:279-288; evaluation counts are summed over ranks."""
    world = 2
    mp.spawn(_net_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / ("net%d.npz" % k)) for k in range(world)]
    seen = [eval(str(z["seen"])) for z in r]
    for s in seen:
        assert [c[0] for c in s] == [5, 5, 5, 2] * 2
        # mask schedule: second epoch, every nb // (H+1) = 1 batch -> perm[0], perm[1], None, None
        assert all(c[2] is None for c in s[:4])
        assert s[4][2] is not None and s[5][2] is not None and s[6][2] is None and s[7][2] is None
    assert [c[2] for c in seen[0]] == [c[2] for c in seen[1]]
    assert all(a[1] != b[1] for a, b in zip(seen[0], seen[1]))  # different slices
    assert int(r[0]["total"][0]) == 2 * (5 + 5 + 5 + 2) == int(r[1]["total"][0])
    assert int(r[0]["correct"][0]) == int(r[1]["correct"][0])
