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


# ---------------------------------------------------------------------------
# The row-sharded layer step (streambrain_b200.parallel.sharded_step) on CPU
# ---------------------------------------------------------------------------
SN, SH, SMC, SB = 300, 3, 4, 5      # 300 rows = 3 tiles of 128: rank 0 owns 256 rows, rank 1 the other 44
SM = SH * SMC
S_HP = dict(taupdt=0.05, khalf=-10.0, pmin=0.1, taubdt=0.1, density=0.5)


def _shard_layer(oracle):
    rng = np.random.RandomState(21)
    layer = oracle.OracleLayer(oracle.PortKernels(), "plastic", SN, SH, SMC, S_HP["taupdt"], (0.5, 1 / SMC, 0.5 / SMC),
                               np.float64, khalf=S_HP["khalf"], pmin=S_HP["pmin"], taubdt=S_HP["taubdt"],
                               density=S_HP["density"], rng=rng)
    layer.Cij = (np.outer(layer.Ci, layer.Cj) * (0.9 + 0.2 * rng.rand(SN, SM)))
    return layer


def _shard_batches(world, steps):
    rs = np.random.RandomState(8)
    return [rs.rand(world * SB, SN) for _ in range(steps)]


class NumpyShardOps:
    """numpy / gloo implementation of the ops protocol of parallel.sharded_step: the layer arithmetic is the
    oracle's, applied to the rows this rank owns; three gathered-input slots used in turn, as in the library."""

    def __init__(self, layer, rank, world, bounds):
        self.layer, self.rank, self.world = layer, rank, world
        self.rb, self.re = bounds[rank]
        self.bounds = bounds
        self.token = torch.zeros(1)
        self.plastic = True
        self.slots, self.cur, self.staged, self.staged_x = [None] * 3, 0, 0, None
        self.calls = []

    def take_staged(self, x):
        if self.staged_x is None:
            return False
        assert self.staged_x is x
        self.staged_x = None
        return True

    def scatter(self, x, ahead):
        parts = [torch.zeros(x.shape[0], SN, dtype=torch.float64) for _ in range(self.world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(x)))
        slot = (self.cur + 1 + self.staged) % 3
        self.staged += 1
        # rank s's samples at rows [s * B, (s + 1) * B), own columns only
        self.slots[slot] = np.concatenate([p.numpy()[:, self.rb:self.re] for p in parts])
        if ahead:
            self.staged_x = x
        self.calls.append(("scatter", ahead, slot))

    def forward(self, x):
        assert self.staged >= 1
        self.cur = (self.cur + 1) % 3
        self.staged -= 1
        self.xg = self.slots[self.cur]
        self.B = x.shape[0]
        self.calls.append(("forward", self.cur))
        return torch.from_numpy(self.xg @ self.layer.weights[self.rb:self.re])

    def join_staged(self):
        self.calls.append(("join",))

    def activate(self, support):
        L = self.layer
        act = support.numpy() + L.bias
        self.yg = L.k.softmax_minicolumns(np.ascontiguousarray(act), SH, SMC)
        self.calls.append(("activate",))
        return self.yg[self.rank * self.B:(self.rank + 1) * self.B]

    def train(self, h):
        L, rb, re = self.layer, self.rb, self.re
        cthr = L.taupdt / 2
        ci, cij, w = L.Ci[rb:re].copy(), L.Cij[rb:re].copy(), L.weights[rb:re].copy()
        _, L.Cj, cij, w = L.k.update_weights(ci, L.Cj, cij, np.ascontiguousarray(self.xg), self.yg, L.taupdt, w, cthr)
        L.Ci[rb:re], L.Cij[rb:re], L.weights[rb:re] = ci, cij, w
        L.bias, L.kbi = L.k.update_bias_regularized(L.bias, L.kbi, L.Cj, cthr, L.khalf, L.pmin, L.taubdt)
        if h is None:   # the masked weights of the own rows (the fused step applies the mask every time)
            L.weights[rb:re] = L.k.apply_mask(np.ascontiguousarray(L.weights[rb:re]),
                                              np.ascontiguousarray(L.wmask[rb:re]), SH, SMC)
        self.calls.append(("train", h))

    def _all_rows(self, a):
        """Every owner's rows of `a`, gathered (stands in for the owners' scores reaching every rank)."""
        width = int(np.prod(a.shape[1:])) if a.ndim > 1 else 1
        rows = max(e - b for b, e in self.bounds)
        mine = np.zeros((rows, width))
        mine[:self.re - self.rb] = a[self.rb:self.re].reshape(self.re - self.rb, width)
        parts = [torch.zeros(rows, width, dtype=torch.float64) for _ in range(self.world)]
        dist.all_gather(parts, torch.from_numpy(mine))
        full = np.concatenate([p.numpy()[:e - b] for p, (b, e) in zip(parts, self.bounds)])
        return full.reshape(a.shape)

    def mask(self, h):
        L, rb, re = self.layer, self.rb, self.re
        cthr = L.taupdt / 2
        Ci, Cij, W = self._all_rows(L.Ci), self._all_rows(L.Cij), self._all_rows(L.weights)
        L.wmask = L.k.update_mask(L.wmask, W, Ci, L.Cj, Cij, cthr, SH, SMC, int(h), 16)
        L.weights[rb:re] = L.k.apply_mask(np.ascontiguousarray(L.weights[rb:re]), np.ascontiguousarray(L.wmask[rb:re]),
                                          SH, SMC)
        self.calls.append(("mask", h))


def _shard_worker(rank, world, port, out_dir):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from streambrain_b200 import parallel
    layer = _shard_layer(oracle)
    bounds = parallel.shard_bounds(SN, world)
    ops = NumpyShardOps(layer, rank, world, bounds)
    batches = _shard_batches(world, 4)
    mine = [xb[rank * SB:(rank + 1) * SB] for xb in batches]
    outs = []
    for k, h in enumerate((1, None, 2, 0)):
        ahead = mine[k + 1] if k in (0, 1) else None    # steps 1 and 2 run on batches staged ahead, step 3 does not
        y = parallel.sharded_step(ops, mine[k], h, lambda t: dist.all_reduce(t, async_op=True), next_x=ahead)
        outs.append(np.array(y))
    rb, re = bounds[rank]
    np.savez(os.path.join(out_dir, "shard%d.npz" % rank), calls=np.array(repr(ops.calls)), y=np.stack(outs),
             Ci=layer.Ci[rb:re], Cij=layer.Cij[rb:re], weights=layer.weights[rb:re], Cj=layer.Cj, bias=layer.bias,
             kbi=layer.kbi, wmask=layer.wmask, rows=np.array([rb, re]))
    dist.destroy_process_group()


def test_two_rank_sharded_step_equals_big_batch(tmp_path):
    """Two gloo ranks run the row-sharded step's orchestration (column exchange, sum of the partial supports,
    every owner updating its rows from the global batch, mask swaps on gathered rows; two of the four batches
    staged one step ahead) and must reproduce the oracle's forward + train step on the whole batches."""
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import oracle
    from streambrain_b200 import parallel
    world = 2
    assert parallel.shard_bounds(SN, world) == [(0, 256), (256, 300)]
    assert parallel.shard_bounds(55296, 8)[7] == (48384, 55296)
    assert parallel.shard_bounds(256, 4) == [(0, 128), (128, 256), (256, 256), (256, 256)]   # more ranks than tiles
    mp.spawn(_shard_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / ("shard%d.npz" % k)) for k in range(world)]
    whole = _shard_layer(oracle)
    ys = []
    for k, (xb, h) in enumerate(zip(_shard_batches(world, 4), (1, None, 2, 0))):
        y = whole.compute_activation(xb)
        whole.train_step(xb, y, h)
        ys.append(y)
    for k in range(world):
        rb, re = r[k]["rows"]
        for step in range(4):
            assert rel_inf(r[k]["y"][step], ys[step][k * SB:(k + 1) * SB]) < 1e-11, (k, step)
        assert np.array_equal(r[k]["wmask"], whole.wmask), k
        for name in ("Ci", "Cij", "weights"):
            assert rel_inf(r[k][name], getattr(whole, name)[rb:re]) < 1e-11, (k, name)
        for name in ("Cj", "bias", "kbi"):
            assert rel_inf(r[k][name], getattr(whole, name)) < 1e-11, (k, name)
            assert np.array_equal(r[k][name], r[0][name]), name      # replicated state stays identical
    calls = eval(str(r[0]["calls"]))
    kinds = [c[0] for c in calls]
    assert kinds == ["scatter", "scatter", "forward", "join", "activate", "train", "mask",     # step 0: own + next
                     "scatter", "forward", "join", "activate", "train",                        # step 1: staged; next
                     "forward", "activate", "train", "mask",                                   # step 2: staged
                     "scatter", "forward", "activate", "train", "mask"]                        # step 3: not staged
    # the gathered-input slots are taken in turn, and a forward pass always takes the oldest staged one
    assert [c[2] for c in calls if c[0] == "scatter"] == [1, 2, 0, 1]
    assert [c[1] for c in calls if c[0] == "forward"] == [1, 2, 0, 1]
