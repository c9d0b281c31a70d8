"""Multi-GPU partitioner for the matmult path (new: the reference has no device or process boundary).

One process per GPU (torch.distributed supplies rank / world size and, where an output has to be
reassembled, the NCCL all-gather).  Two partitionings:

  * batched matmult   -- the batch dimension is split into contiguous ranges, one per rank; items are
                         independent (nt_matmult_batch is a serial loop over items, nt_matmult.hpp:228-235), so
                         there is NO collective on the data path;
  * one large GEMM    -- B (and therefore C) is split by columns, every rank holds all of A; C's column
                         blocks are all-gathered only when the next operation needs full rows.

The arithmetic itself is always this library's kernels on the local shard.
"""
import torch


def shard_range(total, world, rank):
    """Contiguous range [start, start+count) of `total` units owned by `rank`; the first total % world ranks
    get one extra unit, so counts differ by at most one and every unit has exactly one owner."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank %d for world size %d" % (rank, world))
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def column_shard(n, world, rank, align=8):
    """Column range of an n-wide matrix for `rank`, in blocks of `align` columns so every shard keeps
    16-byte aligned rows for 2-byte dtypes (a TMA requirement)."""
    blocks = (n + align - 1) // align
    s, c = shard_range(blocks, world, rank)
    start = s * align
    return start, max(0, min(n, (s + c) * align) - start)


def batched_matmult(a_local, b_local, transpose_a=False, transpose_b=False):
    """Each rank multiplies its own slice of the batch: a plain local call, no communication."""
    from . import api
    return api.matmult(a_local, b_local, transpose_a, transpose_b)


def n_sharded_linear(x, w_local, bias_local=None, group=None, gather=True):
    """y = x.W + b with W split by columns over the ranks of `group`.

    x: [M, K] replicated; w_local: [K, n_r] this rank's columns; returns the full [M, N] (all ranks) when
    `gather`, else the local [M, n_r].  The all-gather is NCCL (or gloo on CPU tensors in host-logic tests);
    column blocks are gathered as [world, M, n_r] and re-tiled to row-major [M, N]."""
    import torch.distributed as dist
    from . import api
    y_local = api.linear(x, w_local, bias_local)
    if not gather or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return y_local
    return all_gather_columns(y_local, group)


def all_gather_columns(y_local, group=None):
    """All-gather equal-width column blocks [M, n_r] of every rank into row-major [M, world * n_r]."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n_r = y_local.shape
    parts = torch.empty((world, m, n_r), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(parts, y_local.contiguous(), group=group)
    return parts.permute(1, 0, 2).reshape(m, world * n_r)
