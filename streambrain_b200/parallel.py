"""Host-side orchestration of the two batch data-parallel train steps: reduce-and-replicate
(``pipelined_dp_step``) and the row-sharded layer (``sharded_step``).

The reference's only parallel scheme is batch data parallelism
(BCPNN/backend/_kernels/kernels_mpi_internal.cc:71-250): every rank forms the
batch sums ``sum_b x``, ``sum_b y`` and ``x^T y`` of its slice, the three are
summed over ranks, and every rank then applies the identical trace / weight
update with divisor ``batch * world_size``.  Here the sums live in one buffer
``delta = [sum_b x (N) | sum_b y (M) | x^T y (N*M)]`` and the row range of
``x^T y`` is cut into blocks so that the reduction of block k overlaps the
product of block k+1.

The functions are written against a small ``ops`` protocol so the same
orchestration runs on CUDA (ops = a device layer, reduction = NCCL) and in CPU
tests (ops = numpy arithmetic, reduction = gloo):

    ops.delta                      1-D tensor of N + M + N*M elements
    ops.n_rows, ops.n_cols         N, M
    ops.local(x, y, rb, re)        fill delta rows [rb, re) (+ the two sums when rb == 0)
    ops.apply_vectors(batch)       Ci, Cj from the reduced sums
    ops.apply_rows(batch, rb, re)  Cij, weights of rows [rb, re)
    ops.finish(h)                  bias and (h is not None) the mask update
"""
from __future__ import annotations


def row_block_bounds(n_rows: int, blocks: int) -> list[tuple[int, int]]:
    """Split [0, n_rows) into at most ``blocks`` ranges whose starts are multiples of 128."""
    tiles = (n_rows + 127) // 128
    blocks = max(1, min(blocks, tiles))
    out, start = [], 0
    for k in range(blocks):
        end = min(n_rows, ((tiles * (k + 1)) // blocks) * 128)
        if end > start:
            out.append((start, end))
            start = end
    return out


def delta_slice(n_rows: int, n_cols: int, rb: int, re: int) -> tuple[int, int]:
    """Element range of ``delta`` that row block [rb, re) owns; block 0 also owns the two sums."""
    lo = 0 if rb == 0 else n_rows + n_cols + rb * n_cols
    return lo, n_rows + n_cols + re * n_cols


def pipelined_dp_step(ops, x, y, hypercolumn, local_batch: int, world_size: int, all_reduce, row_blocks: int = 4):
    """One data-parallel train step.  ``all_reduce(tensor)`` starts an in-place sum
    over ranks and returns a handle with ``wait()`` (``dist.all_reduce(t,
    async_op=True)``)."""
    N, M = ops.n_rows, ops.n_cols
    bounds = row_block_bounds(N, row_blocks)
    works = []
    for rb, re in bounds:
        ops.local(x, y, rb, re)
        lo, hi = delta_slice(N, M, rb, re)
        works.append(all_reduce(ops.delta[lo:hi]))
    batch = local_batch * world_size
    for k, (rb, re) in enumerate(bounds):
        works[k].wait()
        if k == 0:
            ops.apply_vectors(batch)
        ops.apply_rows(batch, rb, re)
    ops.finish(hypercolumn)


def shard_bounds(n_rows: int, world_size: int) -> list[tuple[int, int]]:
    """Input rows [begin, end) each rank of a row-sharded layer owns: equal blocks of whole 128-row
    tiles, the last ones clipped to ``n_rows`` (possibly empty) -- ``sbb_layer_shard_rows``."""
    tiles = (n_rows + 127) // 128
    per = ((tiles + world_size - 1) // world_size) * 128
    return [(min(n_rows, r * per), min(n_rows, (r + 1) * per)) for r in range(world_size)]


def sharded_step(ops, x, hypercolumn, all_reduce, next_x=None, train=True):
    """Forward + train step of a row-sharded, unsupervised layer on this rank's slice ``x`` of the global
    batch; returns the rank's activations.  Every rank owns a block of input rows (``shard_bounds``):
    the ranks exchange the matching columns of their slices, each forms its part of every sample's
    support, ``all_reduce`` sums the parts, and each rank updates its own rows from the whole global
    batch -- the single-device step at the global batch.  With ``next_x`` the exchange of the next
    call's slice is started beside this step's forward product, and this step's all-reduce doubles as
    its barrier.  The ``ops`` protocol (CUDA: the layer's ``sbb_layer_shard_*`` calls; CPU tests: numpy
    over gloo):

        ops.token                  one-element tensor, reduced as a barrier
        ops.plastic                the layer has a mask
        ops.take_staged(x)         True if ``x`` was staged by the previous call (raises on another batch)
        ops.scatter(x, ahead)      exchange the columns of ``x`` (ahead: beside the current step)
        ops.forward(x)             tensor of partial supports of the global batch, to be summed over ranks
        ops.join_staged()          order the step after the exchange started with ahead=True
        ops.activate(support)      bias + softmax; returns this rank's rows
        ops.train(h)               traces and weights of the own rows, bias, (h is not None) mask scores
        ops.mask(h)                the swaps, and the weights of the own swapped rows
    """
    if not ops.take_staged(x):
        ops.scatter(x, False)
        all_reduce(ops.token).wait()
    if next_x is not None:
        ops.scatter(next_x, True)
    support = ops.forward(x)
    if next_x is not None:
        ops.join_staged()
    all_reduce(support).wait()
    y = ops.activate(support)
    if train:
        mask = hypercolumn is not None and ops.plastic
        ops.train(hypercolumn if mask else None)
        if mask:
            all_reduce(ops.token).wait()
            ops.mask(hypercolumn)
    return y


def all_gather_bytes_over(dist):
    """``all_gather_bytes`` for :meth:`shard_rows` on an initialised ``torch.distributed`` group."""
    def gather(blob: bytes):
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, blob)
        return out
    return gather
