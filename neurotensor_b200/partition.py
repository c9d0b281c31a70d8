"""Multi-GPU partitioner for the matmult path (new: the reference has no device or process boundary).

One process per GPU.  The partitioner itself lives behind the C ABI (ntb200_dist_*: shard arithmetic, buffers mapped
into every rank, GEMMs whose epilogues gather their column blocks, a bounded flag exchange for ordering); this module
wraps it for torch processes (torch.distributed supplies rank / world size and carries the buffer records at set-up)
and keeps an NCCL all-gather variant as the comparison baseline.  Two partitionings:

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
    start = min(n, s * align)
    return start, max(0, min(n, (s + c) * align) - start)


def conv2d_image_shard(batch, world, rank):
    """Images of a conv2d batch owned by `rank` (contiguous range).  The convolution of an image depends on no other
    image (functional::conv2d runs one GEMM per image, nt/functional/tensor_files/conv.cpp:69-119), so the forward pass
    and the image gradient need no exchange with the weights replicated; only the kernel gradient, a sum over all
    images, would need an all-reduce of the ranks' partial sums."""
    return shard_range(batch, world, rank)


def sharded_conv2d(x_local, w, stride=1, padding=0, dilation=1, groups=1):
    """conv2d of this rank's images (a plain local call, no communication; weights replicated)."""
    from . import api
    return api.conv2d(x_local, w, stride=stride, padding=padding, dilation=dilation, groups=groups)


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


def c_shard(total, world, rank, align=1):
    """ntb200_dist_shard through the C ABI: (start, count) of `rank`'s contiguous share, in blocks of `align`."""
    import ctypes
    from . import _lib
    s, c = ctypes.c_int64(), ctypes.c_int64()
    _lib.check(_lib.lib().ntb200_dist_shard(total, world, rank, align, ctypes.byref(s), ctypes.byref(c)))
    return s.value, c.value


class DistComm:
    """The library's own communicator (ntb200_dist_* in the C ABI) for the ranks of a torch.distributed group on one
    NVLink domain.  torch.distributed is used once per buffer, at set-up, to pass the 88-byte buffer records around
    (the all-gather callback below); data and ordering afterwards are the library's kernels alone."""

    def __init__(self, group=None):
        import ctypes
        import torch.distributed as dist
        from . import _lib
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

        def exchange(ctx, send, recv, nbytes):
            try:
                mine = ctypes.string_at(send, nbytes)
                parts = [None] * self.world
                dist.all_gather_object(parts, mine, group=group)
                ctypes.memmove(recv, b"".join(parts), nbytes * self.world)
                return 0
            except Exception:                                   # the C side reports the failure
                return 1

        self._cb = _lib.ALLGATHER_FN(exchange)                  # kept alive as long as the communicator
        self._h = ctypes.c_void_p()
        _lib.check(_lib.lib().ntb200_dist_init(ctypes.byref(self._h), self.rank, self.world, self._cb, None))

    def buffer(self, rows, cols, dtype):
        return DistBuffer(self, rows, cols, dtype)

    def barrier(self):
        import ctypes
        from . import _lib
        _lib.check(_lib.lib().ntb200_dist_barrier(self._h, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def gemm_allgather(self, a, b, buf, col0, bias=None, relu=False, row0=0, h_out=None, barrier=True):
        """This rank's column block bias + a.b lands in rows [row0, row0 + m), columns [col0, col0 + n) of `buf` on EVERY
        rank (stored by the GEMM's epilogue), then the ranks are ordered.  relu: returns the pre-activation block [m, n]
        (written into `h_out` when given) and gathers max(., 0); otherwise returns the rows of buf.local it wrote.
        `buf` may belong to another communicator of the same ranks (row blocks gathered on two streams)."""
        import ctypes
        from . import _lib, api
        m, k = a.shape
        n = b.shape[1]
        if row0 < 0 or row0 + m > buf.rows or col0 < 0 or col0 + n > buf.cols or buf.dtype != a.dtype or b.shape[0] != k:
            raise ValueError("gemm_allgather: block [%d x %d] at (%d, %d) does not fit a [%d x %d] buffer" % (m, n, row0, col0, buf.rows, buf.cols))
        d = _lib.GemmDesc()
        d.dtype, d.route, d.accumulate, d.f16_rounding = api.dtype_code(a), _lib.ROUTE_TENSOR, 0, _lib.F16_ROUND_ONCE
        d.m, d.n, d.k, d.batch = m, n, k, 1
        d.a, d.a_row_stride, d.a_col_stride, d.a_batch_stride = a.data_ptr(), a.stride(0), a.stride(1), 0
        d.b, d.b_row_stride, d.b_col_stride, d.b_batch_stride = b.data_ptr(), b.stride(0), b.stride(1), 0
        h = None
        if relu:
            h = h_out if h_out is not None else torch.empty((m, n), dtype=a.dtype, device=a.device)
            if tuple(h.shape) != (m, n) or h.stride(1) != 1 or h.dtype != a.dtype:
                raise ValueError("gemm_allgather: h_out must be a [%d x %d] block with unit column stride" % (m, n))
            d.c, d.c_row_stride, d.c_batch_stride = h.data_ptr(), h.stride(0), 0
        if bias is not None:
            d.bias, d.bias_row_stride, d.bias_col_stride, d.bias_batch_stride = bias.data_ptr(), 0, bias.stride(0), 0
        # barrier=False: no closing flag exchange; the caller orders the ranks (self.barrier()) before anything reads the
        # other ranks' blocks
        entry = _lib.lib().ntb200_dist_gemm_allgather_at if barrier else _lib.lib().ntb200_dist_gemm_push_at
        _lib.check(entry(self._h, ctypes.byref(d), buf._h, buf.cols, row0, col0, int(relu),
                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return h if relu else buf.local[row0:row0 + m]

    def allgather_columns(self, block, buf, col0):
        import ctypes
        from . import _lib, api
        m, n = block.shape
        _lib.check(_lib.lib().ntb200_dist_allgather_columns(self._h, api.dtype_code(block), block.data_ptr(), m, n, block.stride(0),
                                                            buf._h, buf.cols, col0,
                                                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return buf.local

    def close(self):
        from . import _lib
        if self._h is not None:
            _lib.lib().ntb200_dist_destroy(self._h)
            self._h = None


class DistBuffer:
    """A [rows, cols] matrix that exists on every rank of a DistComm and is mapped into every other rank
    (ntb200_dist_buffer_create).  `local` is this rank's copy as a tensor; the peers' copies are only ever written
    by this library's kernels."""

    def __init__(self, comm, rows, cols, dtype):
        import ctypes
        from . import _lib
        self.comm, self.rows, self.cols, self.dtype = comm, rows, cols, dtype
        es = torch.empty((), dtype=dtype).element_size()
        self._h = ctypes.c_void_p()
        _lib.check(_lib.lib().ntb200_dist_buffer_create(comm._h, rows * cols * es, ctypes.byref(self._h)))
        ptr = _lib.lib().ntb200_dist_buffer_ptr(self._h)
        raw = torch.as_tensor(_RawCuda(ptr, (rows, cols * es), "|u1"), device="cuda")
        self.local = raw.view(dtype)

    def close(self):
        from . import _lib
        if self._h is not None:
            self.local = None
            _lib.lib().ntb200_dist_buffer_destroy(self._h)
            self._h = None


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

    def enable_fused_gather(self, batch, comm=None):
        """Switch the two all-gathers to the fused form: the GEMM epilogue stores its column block straight into every
        rank's full buffer (stores into peer-mapped memory), and the library's flag exchange orders the ranks
        (ntb200_dist_gemm_allgather).  Two buffers alternate per step so a fast rank never overwrites what a slower
        rank is still reading."""
        dt = self.w2.dtype
        hidden, dout = self.w2.shape
        own = comm is None
        comm = comm or DistComm(self.group)
        # a second communicator (its own flags) and a side stream for the second row block of step_fused_pipelined
        self._fused = {"comm": comm, "own_comm": own, "more_comms": [DistComm(self.group) for _ in range(3)],
                       "side": [torch.cuda.Stream() for _ in range(3)],
                       "a": [comm.buffer(batch, hidden, dt) for _ in range(2)],
                       "y": [comm.buffer(batch, dout, dt) for _ in range(2)], "parity": 0}

    def close(self):
        f = getattr(self, "_fused", None)
        if f:
            for key in ("a", "y"):
                for b in f[key]:
                    b.close()
            for c in f["more_comms"]:
                c.close()
            if f["own_comm"]:
                f["comm"].close()
        self._fused = None

    def step_fused_pipelined(self, x, target, nblocks=2, early_dw2=False):
        """step_fused with the forward pass in `nblocks` (2 or 4) row blocks, each on a stream of its own: while one
        block's activations cross NVLink the next block is being computed, and layer 2 of a block runs while the later
        blocks' activations travel.  Rows are independent, so every result is bit for bit the one of step_fused; the
        backward pass (which contracts over all rows) is unchanged.  It pays when the gather is longer than the math,
        i.e. from about four GPUs on (at eight, a rank receives 235 MB of activations per step against 0.13 ms of
        layer-1 math).  Every stream has a communicator (flags) of its own; all write into one gathered buffer.
        early_dw2: the gradient of W2's columns needs only this rank's own block of the output (and the gathered
        activations), so it starts as soon as layer 2 has been computed here, on a stream of its own, while the other
        ranks' output blocks are still on the links; its operand is the same gradient block, element for element."""
        from . import api
        f = self._fused
        par = f["parity"]
        f["parity"] ^= 1
        abuf, ybuf = f["a"][par], f["y"][par]
        nblocks = max(1, min(int(nblocks), 1 + len(f["more_comms"])))
        comms = [f["comm"]] + f["more_comms"][:nblocks - 1]
        main = torch.cuda.current_stream()
        streams = [main] + f["side"][:nblocks - 1]
        rows = x.shape[0]
        per = (-(-rows // nblocks) + 127) // 128 * 128
        blocks = [(r0, min(per, rows - r0)) for r0 in range(0, rows, per)]
        h_loc = torch.empty((rows, self.hn), dtype=x.dtype, device=x.device)
        w2_cols = self.w2[:, self.d0:self.d0 + self.dn]
        b2_cols = self.b2[self.d0:self.d0 + self.dn]
        mark = self._mark
        mark("start")
        for st in streams[1:]:
            st.wait_stream(main)
        for i, (r0, nr) in enumerate(blocks):
            with torch.cuda.stream(streams[i]):
                comms[i].gemm_allgather(x[r0:r0 + nr], self.w1, abuf, self.h0, bias=self.b1, relu=True, row0=r0, h_out=h_loc[r0:r0 + nr])
        a, y = abuf.local, ybuf.local
        gw2_loc = gb2_loc = None
        if early_dw2:
            bw = f["side"][-1]
            for i, (r0, nr) in enumerate(blocks):
                with torch.cuda.stream(streams[i]):
                    comms[i].gemm_allgather(a[r0:r0 + nr], w2_cols, ybuf, self.d0, bias=b2_cols, row0=r0, barrier=False)
                bw.wait_stream(streams[i])              # this rank's rows of its own output block are complete
            with torch.cuda.stream(bw):
                dy_blk = api.mse_grad_block(y[:, self.d0:self.d0 + self.dn], target[:, self.d0:self.d0 + self.dn], y.numel())
                gw2_loc = api.matmult(a, dy_blk, True, False)
                gb2_loc = api.column_sum(dy_blk)
            for i in range(len(blocks)):
                with torch.cuda.stream(streams[i]):
                    comms[i].barrier()
            main.wait_stream(bw)
        else:
            for i, (r0, nr) in enumerate(blocks):
                with torch.cuda.stream(streams[i]):
                    comms[i].gemm_allgather(a[r0:r0 + nr], w2_cols, ybuf, self.d0, bias=b2_cols, row0=r0)
        for st in streams[1:]:
            main.wait_stream(st)
        mark("forward: %d row blocks on %d streams, both layers, gathers and flag exchanges%s"
             % (len(blocks), len(blocks), " (dW2, db2 alongside the output gather)" if early_dw2 else ""))
        loss, dy = api.mse(y, target)
        mark("MSE and its gradient")
        if gw2_loc is None:
            dy_loc = dy[:, self.d0:self.d0 + self.dn]
            gw2_loc = api.matmult(a, dy_loc, True, False)
            gb2_loc = api.column_sum(dy_loc.contiguous())
        mark("dW2, db2")
        w2_rows = self.w2[self.h0:self.h0 + self.hn]
        dh_loc = api.matmult_relu_backward(dy, w2_rows, h_loc, True)           # ReLU mask in the epilogue
        mark("dH with the ReLU mask")
        gw1_loc = api.matmult(x, dh_loc, True, False)
        gb1_loc = api.column_sum(dh_loc)
        mark("dW1, db1")
        return loss, dict(w1=gw1_loc, b1=gb1_loc, w2=gw2_loc, b2=gb2_loc, y=y)

    def step_fused(self, x, target):
        """Same step with the all-gathers fused into the GEMM epilogues: layer 1 keeps its pre-activation block and
        stores the activation block into every rank's activation buffer (one launch), layer 2 stores its output
        block; the ranks are ordered after each before anybody reads a gathered buffer.  The backward is the one of
        step()."""
        from . import api
        f = self._fused
        par = f["parity"]
        f["parity"] ^= 1
        comm, abuf, ybuf = f["comm"], f["a"][par], f["y"][par]
        mark = self._mark
        mark("start")
        h_loc = comm.gemm_allgather(x, self.w1, abuf, self.h0, bias=self.b1, relu=True)
        mark("layer 1: GEMM + ReLU, activation block stored into every rank, flag exchange")
        a = abuf.local                                                         # [B, H], every rank's block
        w2_cols = self.w2[:, self.d0:self.d0 + self.dn]
        y = comm.gemm_allgather(a, w2_cols, ybuf, self.d0, bias=self.b2[self.d0:self.d0 + self.dn])
        mark("layer 2: GEMM, output block stored into every rank, flag exchange")
        loss, dy = api.mse(y, target)
        mark("MSE and its gradient")
        dy_loc = dy[:, self.d0:self.d0 + self.dn]
        gw2_loc = api.matmult(a, dy_loc, True, False)
        gb2_loc = api.column_sum(dy_loc.contiguous())
        mark("dW2, db2")
        w2_rows = self.w2[self.h0:self.h0 + self.hn]
        dh_loc = api.matmult_relu_backward(dy, w2_rows, h_loc, True)           # ReLU mask in the epilogue
        mark("dH with the ReLU mask")
        gw1_loc = api.matmult(x, dh_loc, True, False)
        gb1_loc = api.column_sum(dh_loc)
        mark("dW1, db1")
        return loss, dict(w1=gw1_loc, b1=gb1_loc, w2=gw2_loc, b2=gb2_loc, y=y)

    def _mark(self, name):
        """Phase boundary of step_fused: a CUDA event when `phase_events` is a list (bench_mlp_sharded --phases)."""
        ev = getattr(self, "phase_events", None)
        if ev is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            ev.append((name, e))

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
