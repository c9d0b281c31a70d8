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
    """All-gather equal-width column blocks [M, n_r] of every rank into row-major [M, world * n_r].

    The collective gathers whole blocks ([world, M, n_r]); one strided-copy kernel of this library re-tiles them
    into rows (on CPU tensors, used by the host-logic tests, torch does the re-tiling)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n_r = y_local.shape
    parts = torch.empty((world, m, n_r), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(parts.view(world * m, n_r), y_local.contiguous(), group=group)   # rank-major blocks
    if not y_local.is_cuda:
        return parts.permute(1, 0, 2).reshape(m, world * n_r)
    import ctypes
    from . import _lib, api
    out = torch.empty((m, world * n_r), dtype=y_local.dtype, device=y_local.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for m0 in range(0, m, 65535):      # the copy kernel batches over rows: dst[row][rank][:] = parts[rank][row][:]
        mb = min(65535, m - m0)
        _lib.check(_lib.lib().ntb200_copy_strided_2d(api.dtype_code(y_local), out[m0:].data_ptr(), parts[:, m0:].data_ptr(),
                                                     mb, world, n_r, n_r, m * n_r, 1, stream))
    return out


class ShardedMLP:
    """Linear -> ReLU -> Linear -> MSE, forward and backward, with every large GEMM split over the output columns
    (N) across the ranks of a process group.

    Every rank holds x, the target, this rank's columns of W1 / b1, and all of W2 / b2 (its column block is read as a
    strided view for the forward pass, its row block for the backward pass; nothing is copied).  Communication per
    step: one all-gather of the hidden activations and one of the output, both only because the next operation
    needs full rows.  Gradients come out sharded the same way as the parameters they belong to
    (dW1, db1: this rank's columns; dW2, db2: this rank's columns)."""

    def __init__(self, w1_local, b1_local, w2_full, b2_full, rank, world, group=None):
        self.w1, self.b1, self.w2, self.b2 = w1_local, b1_local, w2_full, b2_full
        self.rank, self.world, self.group = rank, world, group
        self.h0, self.hn = column_shard(w2_full.shape[0], world, rank)       # hidden units owned by this rank
        self.d0, self.dn = column_shard(w2_full.shape[1], world, rank)       # output columns owned by this rank
        assert w1_local.shape[1] == self.hn, "W1 shard does not match the hidden partition"

    def gather(self, t):
        if self.world == 1:
            return t
        return all_gather_columns(t, self.group)

    def step(self, x, target):
        from . import api
        h_loc = api.linear(x, self.w1, self.b1)                               # [B, hn]
        a_loc = api.relu(h_loc)
        a = self.gather(a_loc)                                                # [B, H]   all-gather 1
        w2_cols = self.w2[:, self.d0:self.d0 + self.dn]                       # strided view
        y_loc = api.linear(a, w2_cols, self.b2[self.d0:self.d0 + self.dn])    # [B, dn]
        y = self.gather(y_loc)                                                # [B, D]   all-gather 2
        loss, dy = api.mse(y, target)
        dy_loc = dy[:, self.d0:self.d0 + self.dn]                             # strided view
        gw2_loc = api.matmult(a, dy_loc, True, False)                         # [H, dn]
        gb2_loc = api.column_sum(dy_loc.contiguous())
        w2_rows = self.w2[self.h0:self.h0 + self.hn]                          # [hn, D]
        da_loc = api.matmult(dy, w2_rows, False, True)                        # [B, hn]
        dh_loc = api.relu_backward(h_loc, da_loc)
        gw1_loc = api.matmult(x, dh_loc, True, False)                         # [Din, hn]
        gb1_loc = api.column_sum(dh_loc)
        return loss, dict(w1=gw1_loc, b1=gb1_loc, w2=gw2_loc, b2=gb2_loc, y=y)
