"""Host-side orchestration of the batch data-parallel train step.

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


def all_gather_bytes_over(dist):
    """``all_gather_bytes`` for :meth:`shard_rows` on an initialised ``torch.distributed`` group."""
    def gather(blob: bytes):
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, blob)
        return out
    return gather
