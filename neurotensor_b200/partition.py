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


class _RawCuda:
    """A device pointer dressed up for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3}


class PeerBuffer:
    """A [rows, cols] buffer of a 2-byte dtype that exists on every rank and is mapped into every other rank
    (cudaMalloc + CUDA IPC through the library's peer_* entry points).  `local` is this rank's tensor; `peer_bases`
    are raw device pointers of the other ranks' copies, valid for this library's kernels only (they are never handed
    to torch or NCCL)."""

    def __init__(self, rows, cols, dtype, group=None):
        import ctypes
        import torch.distributed as dist
        from . import _lib
        assert dtype in (torch.float16, torch.bfloat16)
        self.rows, self.cols, self.dtype = rows, cols, dtype
        L = _lib.lib()
        ptr = ctypes.c_void_p()
        _lib.check(L.ntb200_peer_alloc(ctypes.byref(ptr), rows * cols * 2))
        self._ptr = ptr
        self.local = torch.as_tensor(_RawCuda(ptr.value, (rows, cols), "<i2"), device="cuda").view(dtype)
        handle = ctypes.create_string_buffer(64)
        _lib.check(L.ntb200_peer_export(ptr, handle))
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self._imported = []
        self.peer_bases = []
        for r in range(world):
            if r == rank:
                continue
            p = ctypes.c_void_p()
            _lib.check(L.ntb200_peer_import(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(p)))
            self._imported.append(p)
            self.peer_bases.append(p.value)

    def close(self):
        from . import _lib
        L = _lib.lib()
        for p in self._imported:
            L.ntb200_peer_release(p)
        self._imported, self.peer_bases = [], []
        if self._ptr is not None:
            self.local = None
            L.ntb200_peer_free(self._ptr)
            self._ptr = None


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

    def enable_fused_gather(self, batch):
        """Switch the two all-gathers to the fused form: the GEMM epilogue stores its column block straight into every
        rank's full buffer (peer stores), and one tiny NCCL all-reduce orders the ranks.  Two buffers alternate per
        step so a fast rank never overwrites what a slower rank is still reading."""
        dt = self.w2.dtype
        hidden, dout = self.w2.shape
        self._fused = {"a": [PeerBuffer(batch, hidden, dt, self.group) for _ in range(2)],
                       "y": [PeerBuffer(batch, dout, dt, self.group) for _ in range(2)],
                       "flag": torch.zeros(1, device="cuda"), "parity": 0}

    def close(self):
        for bufs in (getattr(self, "_fused", None) or {}).values():
            if isinstance(bufs, list):
                for b in bufs:
                    b.close()
        self._fused = None

    def _rank_barrier(self):
        import torch.distributed as dist
        dist.all_reduce(self._fused["flag"], group=self.group)   # stream-ordered: every rank's GEMM is behind it

    def step_fused(self, x, target):
        """Same step with the all-gathers fused into the GEMM epilogues: layer 1 keeps its pre-activation block and
        pushes the activation block into every rank's activation buffer (one launch), layer 2 pushes its output
        block; one barrier after each before anybody reads a gathered buffer.  The backward is the one of step()."""
        from . import api
        f = self._fused
        par = f["parity"]
        f["parity"] ^= 1
        abuf, ybuf = f["a"][par], f["y"][par]
        h_loc = api.gemm_push_relu(x, self.w1, abuf.local, self.h0, bias=self.b1, peer_bases=abuf.peer_bases)
        self._rank_barrier()
        a = abuf.local                                                         # [B, H], every rank's block
        w2_cols = self.w2[:, self.d0:self.d0 + self.dn]
        api.gemm_push(a, w2_cols, ybuf.local, self.d0, bias=self.b2[self.d0:self.d0 + self.dn], peer_bases=ybuf.peer_bases)
        self._rank_barrier()
        y = ybuf.local
        loss, dy = api.mse(y, target)
        dy_loc = dy[:, self.d0:self.d0 + self.dn]
        gw2_loc = api.matmult(a, dy_loc, True, False)
        gb2_loc = api.column_sum(dy_loc.contiguous())
        w2_rows = self.w2[self.h0:self.h0 + self.hn]
        dh_loc = api.matmult_relu_backward(dy, w2_rows, h_loc, True)           # ReLU mask in the epilogue
        gw1_loc = api.matmult(x, dh_loc, True, False)
        gb1_loc = api.column_sum(dh_loc)
        return loss, dict(w1=gw1_loc, b1=gb1_loc, w2=gw2_loc, b2=gb2_loc, y=y)

    def step(self, x, target):
        from . import api
        h_loc, a_loc = api.linear_relu(x, self.w1, self.b1)                   # [B, hn] twice, one launch
        a = self.gather(a_loc)                                                # [B, H]   all-gather 1
        w2_cols = self.w2[:, self.d0:self.d0 + self.dn]                       # strided view
        y_loc = api.linear(a, w2_cols, self.b2[self.d0:self.d0 + self.dn])    # [B, dn]
        y = self.gather(y_loc)                                                # [B, D]   all-gather 2
        loss, dy = api.mse(y, target)
        dy_loc = dy[:, self.d0:self.d0 + self.dn]                             # strided view
        gw2_loc = api.matmult(a, dy_loc, True, False)                         # [H, dn]
        gb2_loc = api.column_sum(dy_loc.contiguous())
        w2_rows = self.w2[self.h0:self.h0 + self.hn]                          # [hn, D]
        dh_loc = api.matmult_relu_backward(dy, w2_rows, h_loc, True)           # [B, hn], ReLU mask in the epilogue
        gw1_loc = api.matmult(x, dh_loc, True, False)                         # [Din, hn]
        gb1_loc = api.column_sum(dh_loc)
        return loss, dict(w1=gw1_loc, b1=gb1_loc, w2=gw2_loc, b2=gb2_loc, y=y)
