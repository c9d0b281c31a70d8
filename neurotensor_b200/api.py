"""Python mirror of the reference's functional interface for the matmult path, on CUDA tensors.

Names, argument meaning and error behaviour follow the reference (paths relative to its project root):

  matmult, matmult_cT, linear   nt/functional/tensor_files/matmult.h:10-13, matmult.cpp:14-38
  shape rules                   nt/functional/cpu/matmult_cpu.cpp:51-93 (determine_transposes), :863-1005 (batches)
  unfold2d / conv2d             nt/functional/tensor_files/colim_transform.cpp:565-588, conv.cpp:69-96
  relu / MSE                    nt/nn/functional/min_max.cpp:40-63, nt/nn/Loss.cpp:49-55
  matmult / linear backward     nt/nn/functional/matmult.cpp:37-63,253-273

A torch.Tensor is used only as a typed handle on device memory (pointer, shape, strides); every operation
is a call through the C ABI of libntb200.so on the current CUDA stream.  Transposed / strided views are
passed as strides and are never copied when one of the last two strides is 1.  Shape and dtype problems
raise ValueError (the reference throws std::invalid_argument) before anything is launched.
"""
import ctypes

import torch

from . import _lib
from ._lib import GemmDesc, check, lib

_TORCH_TO_CODE = {
    torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.int8: _lib.I8,
    torch.int16: _lib.I16, torch.int32: _lib.I32, torch.int64: _lib.I64, torch.float64: _lib.F64,
    torch.uint8: _lib.U8,
    # interleaved (re, im); the reference's componentwise semantics, see NTB200_C64 in include/ntb200.h
    torch.complex64: _lib.C64, torch.complex128: _lib.C128, torch.complex32: _lib.C32,
}


def dtype_code(t):
    try:
        return _TORCH_TO_CODE[t.dtype]
    except KeyError:
        raise ValueError("Expected a number type for matmult but got %s" % t.dtype)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("neurotensor_b200 operates on CUDA tensors only (there is no CPU path)")


def _batch_view(t):
    """(tensor, batch, batch_stride, row_stride, col_stride): leading dims folded into one batch stride.
    A layout whose leading dims cannot be folded is made contiguous first."""
    if t.dim() == 2:
        return t, 1, 0, t.stride(0), t.stride(1)
    lead = t.shape[:-2]
    nb = 1
    for s in lead:
        nb *= s
    # foldable iff stride[i] == stride[i+1] * shape[i+1] over the leading dims
    ok = all(t.stride(i) == t.stride(i + 1) * t.shape[i + 1] for i in range(len(lead) - 1))
    if not ok:
        t = t.contiguous()
    return t, nb, (t.stride(len(lead) - 1) if nb > 1 else 0), t.stride(-2), t.stride(-1)


def _matmult_shapes(a, b, transpose_a, transpose_b):
    if a.dim() < 2 or b.dim() < 2:
        raise ValueError("Expected tensors of at least 2 dims for matmult but got %dD and %dD" % (a.dim(), b.dim()))
    if a.dtype != b.dtype:
        raise ValueError("Expected both tensors to have the same dtype for matmult but got %s and %s"
                         % (a.dtype, b.dtype))
    m, k = (a.shape[-1], a.shape[-2]) if transpose_a else (a.shape[-2], a.shape[-1])
    k2, n = (b.shape[-1], b.shape[-2]) if transpose_b else (b.shape[-2], b.shape[-1])
    if k != k2:
        raise ValueError("Expected second tensor rows to be %d when it was %d (shapes %s and %s, transpose_a=%s, "
                         "transpose_b=%s)" % (k, k2, tuple(a.shape), tuple(b.shape), transpose_a, transpose_b))
    la, lb = tuple(a.shape[:-2]), tuple(b.shape[:-2])
    longer, shorter = (la, lb) if len(la) >= len(lb) else (lb, la)
    if shorter and longer[len(longer) - len(shorter):] != shorter:
        raise ValueError("Expected batch dims to match on the shared suffix but got %s and %s" % (la, lb))
    if shorter and len(shorter) != len(longer):
        raise ValueError("A lower-rank batched operand is not supported; pass a 2-D tensor to repeat it")
    return m, k, n, longer


def gemm(a, b, out, transpose_a=False, transpose_b=False, accumulate=False, bias=None, route=_lib.ROUTE_AUTO,
         f16_rounding=_lib.F16_ROUND_ONCE, relu_out=None, relu_mask=None):
    """out = (accumulate ? out : 0) + bias + op(a).op(b); `out` contiguous in its last dim."""
    _require_cuda(a, b, out, bias)
    m, k, n, lead = _matmult_shapes(a, b, transpose_a, transpose_b)
    if out.dtype != a.dtype:
        raise ValueError("Expected out to have dtype %s but got %s" % (a.dtype, out.dtype))
    if tuple(out.shape) != tuple(lead) + (m, n):
        raise ValueError("Expected out to have shape %s but got %s" % (tuple(lead) + (m, n), tuple(out.shape)))
    if not out.is_contiguous():
        raise ValueError("Expected out to be contiguous")
    av, ab, a_bs, a_rs, a_cs = _batch_view(a)
    bv, bb, b_bs, b_rs, b_cs = _batch_view(b)
    if transpose_a:
        a_rs, a_cs = a_cs, a_rs
    if transpose_b:
        b_rs, b_cs = b_cs, b_rs
    nb = 1
    for s in lead:
        nb *= s
    d = GemmDesc()
    d.dtype, d.route, d.accumulate, d.f16_rounding = dtype_code(a), route, int(bool(accumulate)), f16_rounding
    d.m, d.n, d.k, d.batch = m, n, k, nb
    d.a, d.a_row_stride, d.a_col_stride, d.a_batch_stride = av.data_ptr(), a_rs, a_cs, (a_bs if ab > 1 else 0)
    d.b, d.b_row_stride, d.b_col_stride, d.b_batch_stride = bv.data_ptr(), b_rs, b_cs, (b_bs if bb > 1 else 0)
    d.c, d.c_row_stride, d.c_batch_stride = out.data_ptr(), n, m * n
    if bias is not None:
        if bias.dtype != a.dtype:
            raise ValueError("Expected bias to have dtype %s but got %s" % (a.dtype, bias.dtype))
        try:
            bx = bias.expand(tuple(lead) + (m, n))
        except RuntimeError:
            raise ValueError("bias of shape %s cannot be broadcast to the output %s"
                             % (tuple(bias.shape), tuple(lead) + (m, n)))
        st = bx.stride()
        lead_strides = st[:-2]
        foldable = all(lead_strides[i] == lead_strides[i + 1] * bx.shape[i + 1]
                       for i in range(len(lead_strides) - 1))
        if nb > 1 and any(lead_strides) and not foldable:
            bx = bx.contiguous()
            st = bx.stride()
            lead_strides = st[:-2]
        d.bias = bx.data_ptr()
        d.bias_row_stride, d.bias_col_stride = st[-2], st[-1]
        d.bias_batch_stride = lead_strides[-1] if (nb > 1 and lead_strides) else 0
    for t, name in ((relu_out, "relu_out"), (relu_mask, "relu_mask")):
        if t is not None and (tuple(t.shape) != tuple(out.shape) or t.dtype != out.dtype or not t.is_contiguous() or not t.is_cuda):
            raise ValueError("%s must be a contiguous CUDA tensor shaped and typed like the output" % name)
    if relu_out is not None or relu_mask is not None:
        ep = _lib.GemmEpilogue()
        ep.relu_out = relu_out.data_ptr() if relu_out is not None else None
        ep.relu_mask_src = relu_mask.data_ptr() if relu_mask is not None else None
        check(lib().ntb200_gemm_fused(ctypes.byref(d), ctypes.byref(ep), _stream()))
    else:
        check(lib().ntb200_gemm(ctypes.byref(d), _stream()))
    return out


def linear_relu(x, w, bias=None):
    """h = x.w + bias and a = relu(h) from ONE launch (the ReLU is a second output of the GEMM epilogue).  Falls back
    to two launches when the tensor-core route cannot take the operands."""
    m, k, n, lead = _matmult_shapes(x, w, False, False)
    h = torch.empty(tuple(lead) + (m, n), dtype=x.dtype, device=x.device)
    if x.dtype in (torch.float16, torch.bfloat16):
        a = torch.empty_like(h)
        try:
            gemm(x, w, h, bias=bias, relu_out=a)
            return h, a
        except _lib.Ntb200Error as e:
            if e.code != _lib.ERR_UNSUPPORTED:
                raise
    gemm(x, w, h, bias=bias)
    return h, relu(h)


def matmult_relu_backward(grad, w, h, transpose_b=True):
    """dH = relu_backward(h, grad . op(w)) from ONE launch: the clamp mask is applied in the GEMM epilogue."""
    m, k, n, lead = _matmult_shapes(grad, w, False, transpose_b)
    out = torch.empty(tuple(lead) + (m, n), dtype=grad.dtype, device=grad.device)
    if grad.dtype in (torch.float16, torch.bfloat16) and h.is_contiguous():
        try:
            return gemm(grad, w, out, False, transpose_b, relu_mask=h)
        except _lib.Ntb200Error as e:
            if e.code != _lib.ERR_UNSUPPORTED:
                raise
    gemm(grad, w, out, False, transpose_b)
    return relu_backward(h, out)


def gemm_push(a, b, full_out, col0, bias=None, transpose_a=False, transpose_b=False, peer_bases=()):
    """full_out[:, col0:col0+n] = bias + op(a).op(b), and the same block into the buffers at `peer_bases` (raw device
    pointers of peer-mapped tensors shaped like `full_out` on other GPUs): the column all-gather of an N-sharded GEMM
    done by the GEMM's own epilogue.  2-D, Float16 / BFloat16, tensor-core route."""
    _require_cuda(a, b, full_out, bias)
    m, k, n, lead = _matmult_shapes(a, b, transpose_a, transpose_b)
    if lead or full_out.dim() != 2 or not full_out.is_contiguous():
        raise ValueError("gemm_push takes 2-D operands and a contiguous 2-D output buffer")
    if full_out.shape[0] != m or col0 < 0 or col0 + n > full_out.shape[1] or full_out.dtype != a.dtype:
        raise ValueError("gemm_push: column block [%d, %d) does not fit an output of shape %s" % (col0, col0 + n, tuple(full_out.shape)))
    es = full_out.element_size()
    a_rs, a_cs = (a.stride(1), a.stride(0)) if transpose_a else (a.stride(0), a.stride(1))
    b_rs, b_cs = (b.stride(1), b.stride(0)) if transpose_b else (b.stride(0), b.stride(1))
    d = GemmDesc()
    d.dtype, d.route, d.accumulate, d.f16_rounding = dtype_code(a), _lib.ROUTE_TENSOR, 0, _lib.F16_ROUND_ONCE
    d.m, d.n, d.k, d.batch = m, n, k, 1
    d.a, d.a_row_stride, d.a_col_stride, d.a_batch_stride = a.data_ptr(), a_rs, a_cs, 0
    d.b, d.b_row_stride, d.b_col_stride, d.b_batch_stride = b.data_ptr(), b_rs, b_cs, 0
    d.c, d.c_row_stride, d.c_batch_stride = full_out.data_ptr() + col0 * es, full_out.shape[1], 0
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != n or bias.dtype != a.dtype:
            raise ValueError("gemm_push: bias must be a vector of the block's %d columns" % n)
        d.bias, d.bias_row_stride, d.bias_col_stride, d.bias_batch_stride = bias.data_ptr(), 0, bias.stride(0), 0
    peers = (ctypes.c_void_p * max(1, len(peer_bases)))(*[int(p) + col0 * es for p in peer_bases])
    check(lib().ntb200_gemm_push(ctypes.byref(d), peers, len(peer_bases), _stream()))
    return full_out


def gemm_push_relu(a, b, full_act, col0, bias=None, peer_bases=()):
    """Linear + ReLU of one rank's column block of an N-sharded layer, gathered by the GEMM itself:
    h = bias + a.b is returned (contiguous [m, n], kept for the backward mask) and max(h, 0) is written to
    full_act[:, col0:col0+n] here and at the same place in the peer-mapped buffers at `peer_bases`.  One launch."""
    _require_cuda(a, b, full_act, bias)
    m, k, n, lead = _matmult_shapes(a, b, False, False)
    if lead or full_act.dim() != 2 or not full_act.is_contiguous():
        raise ValueError("gemm_push_relu takes 2-D operands and a contiguous 2-D activation buffer")
    if full_act.shape[0] != m or col0 < 0 or col0 + n > full_act.shape[1] or full_act.dtype != a.dtype:
        raise ValueError("gemm_push_relu: column block [%d, %d) does not fit a buffer of shape %s"
                         % (col0, col0 + n, tuple(full_act.shape)))
    es = full_act.element_size()
    h = torch.empty((m, n), dtype=a.dtype, device=a.device)
    d = GemmDesc()
    d.dtype, d.route, d.accumulate, d.f16_rounding = dtype_code(a), _lib.ROUTE_TENSOR, 0, _lib.F16_ROUND_ONCE
    d.m, d.n, d.k, d.batch = m, n, k, 1
    d.a, d.a_row_stride, d.a_col_stride, d.a_batch_stride = a.data_ptr(), a.stride(0), a.stride(1), 0
    d.b, d.b_row_stride, d.b_col_stride, d.b_batch_stride = b.data_ptr(), b.stride(0), b.stride(1), 0
    d.c, d.c_row_stride, d.c_batch_stride = h.data_ptr(), n, 0
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != n or bias.dtype != a.dtype:
            raise ValueError("gemm_push_relu: bias must be a vector of the block's %d columns" % n)
        d.bias, d.bias_row_stride, d.bias_col_stride, d.bias_batch_stride = bias.data_ptr(), 0, bias.stride(0), 0
    peers = (ctypes.c_void_p * max(1, len(peer_bases)))(*[int(p) + col0 * es for p in peer_bases])
    check(lib().ntb200_gemm_push_relu(ctypes.byref(d), full_act.data_ptr() + col0 * es, full_act.shape[1], peers,
                                      len(peer_bases), _stream()))
    return h


def matmult(a, b, transpose_a=False, transpose_b=False, out=None, route=_lib.ROUTE_AUTO,
            f16_rounding=_lib.F16_ROUND_ONCE):
    """functional::matmult.  Without `out` returns a new tensor op(a).op(b); with `out` computes
    out += op(a).op(b) into the caller's contiguous tensor and returns it (matmult_cpu.cpp:137-153)."""
    m, k, n, lead = _matmult_shapes(a, b, transpose_a, transpose_b)
    if out is None:
        res = torch.empty(tuple(lead) + (m, n), dtype=a.dtype, device=a.device)
        return gemm(a, b, res, transpose_a, transpose_b, accumulate=False, route=route, f16_rounding=f16_rounding)
    return gemm(a, b, out, transpose_a, transpose_b, accumulate=True, route=route, f16_rounding=f16_rounding)


def matmult_tensors(a_list, b_list, transpose_a=False, transpose_b=False):
    """functional::matmult on two tensors of tensors (DType::TensorObj operands, matmult_cpu.cpp:1240-1558): two lists
    of the same length, every tensor of a list with one shape and dtype; item i of the result is
    matmult(a_list[i], b_list[i]).  The items may have batch dimensions of their own, and the items of one list may
    have fewer dimensions than those of the other (they are then reused over the other's batch dimensions, the
    reference's `n_k` / `k_n` forms).  Every (item, batch) pair becomes one entry of the pointer tables of a single
    ntb200_matmult_batch call: equally spaced pointers (lists made by splitting one tensor) run as one strided
    launch, anything else through device pointer tables.  Returns the list of results, views of one allocation.
    Errors follow subT_check (matmult_cpu.cpp:1486-1513)."""
    a_list, b_list = list(a_list), list(b_list)
    if len(a_list) != len(b_list):
        raise ValueError("Expected both tensors to have the same number of sub-tensors, going to have these multiplied in a "
                         "list-like fashion, but got %d and %d tensors" % (len(a_list), len(b_list)))
    if not a_list:
        return []
    for name, lst in (("a", a_list), ("b", b_list)):
        for t in lst[1:]:
            if t.shape != lst[0].shape:
                raise ValueError("Expected all tensors in list of tensors to have the same shape, but %s has a tensor of shape "
                                 "%s and %s" % (name, tuple(lst[0].shape), tuple(t.shape)))
            if t.dtype != lst[0].dtype:
                raise ValueError("Expected all tensors in list of tensors to have the same dtype, but %s has a tensor of dtype "
                                 "%s and %s" % (name, lst[0].dtype, t.dtype))
    if a_list[0].dtype != b_list[0].dtype:
        raise ValueError("Expected all tensors in list of tensors to have the same dtype (%s), but b has a tensor of dtype %s"
                         % (a_list[0].dtype, b_list[0].dtype))
    _require_cuda(*a_list, *b_list)
    a0, b0 = a_list[0], b_list[0]
    if a0.dim() < 2 or b0.dim() < 2:
        raise ValueError("matmult: the tensors of a tensor of tensors need at least two dimensions")
    a_rows, a_cols = int(a0.shape[-2]), int(a0.shape[-1])
    b_rows, b_cols = int(b0.shape[-2]), int(b0.shape[-1])
    lead_a, lead_b = tuple(a0.shape[:-2]), tuple(b0.shape[:-2])
    if len(lead_a) >= len(lead_b):
        lead = lead_a
        if lead_b and lead_a[len(lead_a) - len(lead_b):] != lead_b:
            raise ValueError("matmult: batch dimensions %s and %s do not match" % (lead_a, lead_b))
    else:
        lead = lead_b
        if lead_a and lead_b[len(lead_b) - len(lead_a):] != lead_a:
            raise ValueError("matmult: batch dimensions %s and %s do not match" % (lead_a, lead_b))
    inner = 1
    for d in lead:
        inner *= int(d)
    m = a_cols if transpose_a else a_rows
    k = a_rows if transpose_a else a_cols
    kb = b_cols if transpose_b else b_rows
    n = b_rows if transpose_b else b_cols
    if k != kb:
        raise ValueError("Expected second tensor rows to be %d when it was %d" % (k, kb))
    a_list = [t.contiguous() for t in a_list]
    b_list = [t.contiguous() for t in b_list]
    out = torch.zeros((len(a_list),) + lead + (m, n), dtype=a0.dtype, device=a0.device)   # the raw contract is C +=
    es = a0.element_size()
    count = len(a_list) * inner
    pa, pb, pc = (ctypes.c_void_p * count)(), (ctypes.c_void_p * count)(), (ctypes.c_void_p * count)()
    a_inner = a0.numel() // (a_rows * a_cols)
    b_inner = b0.numel() // (b_rows * b_cols)
    for i, (ta, tb) in enumerate(zip(a_list, b_list)):
        base_a, base_b, base_c = ta.data_ptr(), tb.data_ptr(), out[i].data_ptr()
        for j in range(inner):
            pa[i * inner + j] = base_a + (j % a_inner) * a_rows * a_cols * es
            pb[i * inner + j] = base_b + (j % b_inner) * b_rows * b_cols * es
            pc[i * inner + j] = base_c + j * m * n * es
    # the raw contract takes the logical extents of op(a) and op(b); the flags say how they are stored
    check(lib().ntb200_matmult_batch(dtype_code(a0), pa, pb, pc, count, m, k, k, n,
                                     int(bool(transpose_a)), int(bool(transpose_b)), _stream()))
    return [out[i] for i in range(len(a_list))]


def hodge_laplacian_from_boundaries(boundary_kp1, boundary_k=None):
    """The matmult calls of the TDA Hodge Laplacian (nt/tda/nn/laplacian.cpp:42-45,61-62,84-86):
    L = B_{k+1} B_{k+1}^T (+ B_k^T B_k), both products by transpose flags on the boundary matrices, then one
    elementwise add of the two finished products (not a continued accumulation: the reference adds two tensors)."""
    up = matmult(boundary_kp1, boundary_kp1, False, True)
    if boundary_k is None:
        return up
    down = matmult(boundary_k, boundary_k, True, False)
    check(lib().ntb200_add_inplace(dtype_code(up), up.data_ptr(), down.data_ptr(), up.numel(), _stream()))
    return up


def matmult_cT(a, b):
    return matmult(a, b, False, True)


def linear(x, w, bias=None, transpose_a=False, transpose_b=False, route=_lib.ROUTE_AUTO):
    """functional::linear: op(x).op(w) + bias, the bias broadcast over rows and batch."""
    if bias is None:
        return matmult(x, w, transpose_a, transpose_b, route=route)
    m, k, n, lead = _matmult_shapes(x, w, transpose_a, transpose_b)
    res = torch.empty(tuple(lead) + (m, n), dtype=x.dtype, device=x.device)
    return gemm(x, w, res, transpose_a, transpose_b, accumulate=False, bias=bias, route=route)


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _conv_geom(x, kernel_size, dilation, padding, stride):
    kh, kw = _pair(kernel_size)
    dh, dw = _pair(dilation)
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    if sh < 1 or sw < 1:
        raise ValueError("Conv2d stride cannot be less than 1 but got %s" % (stride,))
    if dh < 1 or dw < 1:
        raise ValueError("Conv2d dilation cannot be less than 1 but got %s" % (dilation,))
    if ph < 0 or pw < 0:
        raise ValueError("Conv2d padding cannot be less than 0 but got %s" % (padding,))
    if x.dim() < 3:
        raise ValueError("Expected input tensor to have dims greater than or equal to 3 but got %dD" % x.dim())
    x4 = x.reshape((-1,) + tuple(x.shape[-3:])).contiguous()
    ho = (x4.shape[-2] + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (x4.shape[-1] + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    if ho <= 0 or wo <= 0:
        raise ValueError("calculated shape of the array of sliding blocks as (%d, %d), but its components must be "
                         "at least one" % (ho, wo))
    return x4, (kh, kw, sh, sw, ph, pw, dh, dw), ho, wo


def unfold2d(x, kernel_size, dilation=1, padding=0, stride=1):
    """functional::unfold2d(..., transpose_out=true) -> [B, C*kh*kw, L]."""
    _require_cuda(x)
    x4, (kh, kw, sh, sw, ph, pw, dh, dw), ho, wo = _conv_geom(x, kernel_size, dilation, padding, stride)
    bsz, ch, h, w = x4.shape
    col = torch.empty((bsz, ch * kh * kw, ho * wo), dtype=x.dtype, device=x.device)
    check(lib().ntb200_im2col(dtype_code(x), x4.data_ptr(), col.data_ptr(), bsz, ch, h, w, kh, kw, sh, sw, ph, pw,
                              dh, dw, _stream()))
    return col


def unfold2d_backward(dcol, out_hw, kernel_size, dilation=1, padding=0, stride=1):
    _require_cuda(dcol)
    kh, kw = _pair(kernel_size)
    dh, dw = _pair(dilation)
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    h, w = out_hw
    dcol = dcol.contiguous()
    bsz, ch = dcol.shape[0], dcol.shape[1] // (kh * kw)
    im = torch.empty((bsz, ch, h, w), dtype=dcol.dtype, device=dcol.device)
    check(lib().ntb200_col2im(dtype_code(dcol), dcol.data_ptr(), im.data_ptr(), bsz, ch, h, w, kh, kw, sh, sw, ph, pw,
                              dh, dw, _stream()))
    return im


def _conv_weights(x, w, groups, what="conv2d"):
    if w.dim() not in (3, 4):
        raise ValueError("Expected to get a 4D or 3D tensor as the kernel for a 2d convolution, but got %dD" % w.dim())
    if x.dtype != w.dtype:
        raise ValueError("Expected both kernel and image to have the same dtype for %s but got %s and %s"
                         % (what, w.dtype, x.dtype))
    if groups < 1:
        raise ValueError("Expected groups for a convolution to be greater than 0 but got %d" % groups)
    return (w.unsqueeze(0) if w.dim() == 3 else w).contiguous()


def _grouped_workspace(code, bsz, ch, h, wd, cout, geom, groups, workspace, device):
    kh, kw, sh, sw, ph, pw, dh, dw = geom
    need = lib().ntb200_conv2d_grouped_workspace_bytes(code, bsz, ch, h, wd, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
    return workspace


def conv2d(x, w, stride=1, padding=0, dilation=1, groups=1, workspace=None):
    """functional::conv2d (conv.cpp:69-119) -> [B, Cout, Ho, Wo]; w is [Cout, C/groups, kh, kw]."""
    _require_cuda(x, w)
    w4 = _conv_weights(x, w, groups)
    x4, geom, ho, wo = _conv_geom(x, w4.shape[-2:], dilation, padding, stride)
    kh, kw, sh, sw, ph, pw, dh, dw = geom
    bsz, ch, h, wd = x4.shape
    if ch % groups:
        raise ValueError("Expected image channels to be divisible by groups in Conv2d but got %d %% %d != 0" % (ch, groups))
    if w4.shape[1] * groups != ch:
        raise ValueError("Expected kernel channels %d times groups %d to equal image channels %d" % (w4.shape[1], groups, ch))
    cout = w4.shape[0]
    code = dtype_code(x)
    out = torch.empty((bsz, cout, ho, wo), dtype=x.dtype, device=x.device)
    if groups == 1:
        need = lib().ntb200_conv2d_workspace_bytes(code, bsz, ch, h, wd, kh, kw, sh, sw, ph, pw, dh, dw)
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
        check(lib().ntb200_conv2d(code, x4.data_ptr(), w4.data_ptr(), out.data_ptr(), workspace.data_ptr(), bsz, ch, h,
                                  wd, cout, kh, kw, sh, sw, ph, pw, dh, dw, _stream()))
        return out
    workspace = _grouped_workspace(code, bsz, ch, h, wd, cout, geom, groups, workspace, x.device)
    check(lib().ntb200_conv2d_grouped(code, x4.data_ptr(), w4.data_ptr(), out.data_ptr(), workspace.data_ptr(), bsz, ch, h,
                                      wd, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, _stream()))
    return out


def conv2d_backward(x, w, grad, stride=1, padding=0, dilation=1, groups=1, workspace=None):
    """conv_dimage (conv.cpp:318-346) and conv_dkernel (conv.cpp:444-471) -> (d_image, d_kernel):
    d_image = col2im(matmult(w2d, grad, true, false)); d_kernel = sum over the batch of matmult(grad, col, false, true),
    group by group when groups > 1.  Both run inside the library on one shared workspace."""
    _require_cuda(x, w, grad)
    if not (x.dtype == w.dtype == grad.dtype):
        raise ValueError("conv2d_backward: image, kernel and gradient must share a dtype")
    w4 = _conv_weights(x, w, groups)
    x4, geom, ho, wo = _conv_geom(x, w4.shape[-2:], dilation, padding, stride)
    kh, kw, sh, sw, ph, pw, dh, dw = geom
    x4 = x4.contiguous()
    bsz, ch, h, wd = x4.shape
    cout = w4.shape[0]
    g = grad.contiguous()
    if g.numel() != bsz * cout * ho * wo:
        raise ValueError("conv2d_backward: gradient has %d elements, expected [%d, %d, %d, %d]"
                         % (g.numel(), bsz, cout, ho, wo))
    code = dtype_code(x)
    workspace = _grouped_workspace(code, bsz, ch, h, wd, cout, geom, groups, workspace, x.device)
    dx = torch.empty_like(x4)
    dw_ = torch.empty_like(w4)
    check(lib().ntb200_conv2d_grouped_backward_image(code, g.data_ptr(), w4.data_ptr(), dx.data_ptr(), workspace.data_ptr(),
                                                     bsz, ch, h, wd, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, _stream()))
    check(lib().ntb200_conv2d_grouped_backward_kernel(code, x4.data_ptr(), g.data_ptr(), dw_.data_ptr(), workspace.data_ptr(),
                                                      0, bsz, ch, h, wd, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, _stream()))
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def conv1d(x, w, stride=1, padding=0, dilation=1, groups=1):
    """functional::conv1d (conv.cpp:13-67): [B, C, W] * [Cout, C/groups, k] as the one-row case of conv2d."""
    if x.dim() < 2 or w.dim() not in (2, 3):
        raise ValueError("Expected a 2D or greater input and a 2D or 3D kernel for a 1d convolution")
    w3 = w.unsqueeze(0) if w.dim() == 2 else w
    x3 = x.reshape((-1,) + tuple(x.shape[-2:]))
    out = conv2d(x3.unsqueeze(-2), w3.unsqueeze(-2), (1, stride), (0, padding), (1, dilation), groups)
    return out.squeeze(-2)


def conv1d_backward(x, w, grad, stride=1, padding=0, dilation=1, groups=1):
    w3 = w.unsqueeze(0) if w.dim() == 2 else w
    x3 = x.reshape((-1,) + tuple(x.shape[-2:]))
    g3 = grad.reshape((x3.shape[0], w3.shape[0], -1))
    dx, dw_ = conv2d_backward(x3.unsqueeze(-2), w3.unsqueeze(-2), g3.unsqueeze(-2), (1, stride), (0, padding), (1, dilation),
                              groups)
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def _transpose_geom(x, w4, stride, padding, output_padding, dilation, groups):
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    oh, ow = _pair(output_padding)
    dh, dw = _pair(dilation)
    if sh < 1 or sw < 1:
        raise ValueError("Conv2d Transpose stride cannot be less than 1 but got %s" % (stride,))
    if dh < 1 or dw < 1:
        raise ValueError("Conv2d Transpose dilation cannot be less than 1 but got %s" % (dilation,))
    if ph < 0 or pw < 0 or oh < 0 or ow < 0:
        raise ValueError("Conv2d Transpose padding and output_padding cannot be less than 0")
    if oh >= sh or ow >= sw:
        raise ValueError("conv_transpose2d: output_padding must be smaller than the stride")
    x4 = x.reshape((-1,) + tuple(x.shape[-3:])).contiguous()
    if x4.shape[1] != w4.shape[0]:
        raise ValueError("Expected image channels to be the same as the kernel batches for conv_transpose2d but got %s and %s"
                         % (tuple(x4.shape), tuple(w4.shape)))
    kh, kw = w4.shape[-2:]
    ho = (x4.shape[-2] - 1) * sh - 2 * ph + dh * (kh - 1) + 1 + oh
    wo = (x4.shape[-1] - 1) * sw - 2 * pw + dw * (kw - 1) + 1 + ow
    return x4, (kh, kw, sh, sw, ph, pw, dh, dw), ho, wo


def conv_transpose2d(x, w, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    """functional::conv_transpose2d (conv.cpp:614-672): x [B, Cin, Hi, Wi], w [Cin, Cout/groups, kh, kw] ->
    [B, Cout, Ho, Wo].  It is the image gradient of the convolution that maps [B, Cout, Ho, Wo] to x's shape with
    the same kernel, so it runs as ntb200_conv2d_grouped_backward_image with x in the place of the gradient."""
    _require_cuda(x, w)
    w4 = _conv_weights(x, w, groups, "conv2d transpose")
    x4, geom, ho, wo = _transpose_geom(x, w4, stride, padding, output_padding, dilation, groups)
    kh, kw, sh, sw, ph, pw, dh, dw = geom
    bsz, cin, hi, wi = x4.shape
    cout = w4.shape[1] * groups
    code = dtype_code(x)
    workspace = _grouped_workspace(code, bsz, cout, ho, wo, cin, geom, groups, None, x.device)
    out = torch.empty((bsz, cout, ho, wo), dtype=x.dtype, device=x.device)
    check(lib().ntb200_conv2d_grouped_backward_image(code, x4.data_ptr(), w4.data_ptr(), out.data_ptr(), workspace.data_ptr(),
                                                     bsz, cout, ho, wo, cin, kh, kw, sh, sw, ph, pw, dh, dw, groups, _stream()))
    return out


def conv_transpose2d_backward(x, w, grad, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    """Gradients of conv_transpose2d -> (d_x, d_w): d_x is the forward convolution of grad with w; d_w is the kernel
    gradient of that convolution with the roles of image (grad) and gradient (x) exchanged."""
    _require_cuda(x, w, grad)
    w4 = _conv_weights(x, w, groups, "conv2d transpose")
    x4, geom, ho, wo = _transpose_geom(x, w4, stride, padding, output_padding, dilation, groups)
    kh, kw, sh, sw, ph, pw, dh, dw = geom
    bsz, cin, hi, wi = x4.shape
    cout = w4.shape[1] * groups
    g = grad.contiguous().reshape(bsz, cout, ho, wo)
    code = dtype_code(x)
    workspace = _grouped_workspace(code, bsz, cout, ho, wo, cin, geom, groups, None, x.device)
    dx = torch.empty_like(x4)
    dw_ = torch.empty_like(w4)
    check(lib().ntb200_conv2d_grouped(code, g.data_ptr(), w4.data_ptr(), dx.data_ptr(), workspace.data_ptr(), bsz, cout, ho,
                                      wo, cin, kh, kw, sh, sw, ph, pw, dh, dw, groups, _stream()))
    check(lib().ntb200_conv2d_grouped_backward_kernel(code, g.data_ptr(), x4.data_ptr(), dw_.data_ptr(), workspace.data_ptr(),
                                                      0, bsz, cout, ho, wo, cin, kh, kw, sh, sw, ph, pw, dh, dw, groups, _stream()))
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def conv_transpose1d(x, w, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    """functional::conv_transpose1d (conv.cpp:538-612) as the one-row case of conv_transpose2d."""
    w3 = w.unsqueeze(0) if w.dim() == 2 else w
    x3 = x.reshape((-1,) + tuple(x.shape[-2:]))
    out = conv_transpose2d(x3.unsqueeze(-2), w3.unsqueeze(-2), (1, stride), (0, padding), (0, output_padding), (1, dilation),
                           groups)
    return out.squeeze(-2)


def conv_transpose1d_backward(x, w, grad, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    w3 = w.unsqueeze(0) if w.dim() == 2 else w
    x3 = x.reshape((-1,) + tuple(x.shape[-2:]))
    g3 = grad.reshape((x3.shape[0], -1, grad.shape[-1]))
    dx, dw_ = conv_transpose2d_backward(x3.unsqueeze(-2), w3.unsqueeze(-2), g3.unsqueeze(-2), (1, stride), (0, padding),
                                        (0, output_padding), (1, dilation), groups)
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def _triple(v):
    if isinstance(v, (tuple, list)):
        if len(v) != 3:
            raise ValueError("expected one value or three (depth, height, width), got %r" % (v,))
        return tuple(int(q) for q in v)
    return (int(v),) * 3


def _geom3(bsz, ch, dhw, cout, groups, kernel, stride, padding, dilation):
    g = _lib.Conv3dGeom()
    g.batch, g.channels, (g.depth, g.height, g.width), g.cout, g.groups = bsz, ch, dhw, cout, groups
    for name, val in (("kernel", kernel), ("stride", stride), ("padding", padding), ("dilation", dilation)):
        arr = getattr(g, name)
        for i in range(3):
            arr[i] = val[i]
    return g


def _conv3d_setup(x, w, stride, padding, dilation, groups, what="conv3d"):
    _require_cuda(x, w)
    if x.dim() < 4 or w.dim() not in (4, 5):
        raise ValueError("Expected a 4D or greater input and a 4D or 5D kernel for a 3d convolution")
    if x.dtype != w.dtype:
        raise ValueError("Expected both kernel and image to have the same dtype for %s but got %s and %s" % (what, w.dtype, x.dtype))
    w5 = (w.unsqueeze(0) if w.dim() == 4 else w).contiguous()
    x5 = x.reshape((-1,) + tuple(x.shape[-4:])).contiguous()
    return x5, w5, _triple(stride), _triple(padding), _triple(dilation)


def _out3(size, k, s, p, d):
    return tuple((size[i] + 2 * p[i] - d[i] * (k[i] - 1) - 1) // s[i] + 1 for i in range(3))


def conv3d(x, w, stride=1, padding=0, dilation=1, groups=1):
    """functional::conv3d (conv.cpp:122-174) -> [B, Cout, Do, Ho, Wo]; w is [Cout, C/groups, kd, kh, kw]."""
    x5, w5, s3, p3, d3 = _conv3d_setup(x, w, stride, padding, dilation, groups)
    bsz, ch = x5.shape[:2]
    cout, k3 = w5.shape[0], tuple(w5.shape[-3:])
    if groups < 1 or ch % groups or w5.shape[1] * groups != ch:
        raise ValueError("Expected kernel channels %d times groups %d to equal image channels %d" % (w5.shape[1], groups, ch))
    o3 = _out3(tuple(x5.shape[-3:]), k3, s3, p3, d3)
    if min(o3) <= 0:
        raise ValueError("conv3d: calculated output size %s must be at least one" % (o3,))
    geom = _geom3(bsz, ch, tuple(x5.shape[-3:]), cout, groups, k3, s3, p3, d3)
    code = dtype_code(x)
    ws = torch.empty(max(1, lib().ntb200_conv3d_workspace_bytes(code, ctypes.byref(geom))), dtype=torch.uint8, device=x.device)
    out = torch.empty((bsz, cout) + o3, dtype=x.dtype, device=x.device)
    check(lib().ntb200_conv3d(code, x5.data_ptr(), w5.data_ptr(), out.data_ptr(), ws.data_ptr(), ctypes.byref(geom), _stream()))
    return out


def conv3d_backward(x, w, grad, stride=1, padding=0, dilation=1, groups=1):
    """conv_dimage / conv_dkernel for the 3-D case -> (d_image, d_kernel)."""
    x5, w5, s3, p3, d3 = _conv3d_setup(x, w, stride, padding, dilation, groups)
    _require_cuda(grad)
    bsz, ch = x5.shape[:2]
    cout, k3 = w5.shape[0], tuple(w5.shape[-3:])
    geom = _geom3(bsz, ch, tuple(x5.shape[-3:]), cout, groups, k3, s3, p3, d3)
    code = dtype_code(x)
    g = grad.contiguous()
    ws = torch.empty(max(1, lib().ntb200_conv3d_workspace_bytes(code, ctypes.byref(geom))), dtype=torch.uint8, device=x.device)
    dx, dw_ = torch.empty_like(x5), torch.empty_like(w5)
    check(lib().ntb200_conv3d_backward_image(code, g.data_ptr(), w5.data_ptr(), dx.data_ptr(), ws.data_ptr(), ctypes.byref(geom),
                                             _stream()))
    check(lib().ntb200_conv3d_backward_kernel(code, x5.data_ptr(), g.data_ptr(), dw_.data_ptr(), ws.data_ptr(), 0,
                                              ctypes.byref(geom), _stream()))
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def _transpose3_geom(x5, w5, s3, p3, o3pad, d3, groups):
    if x5.shape[1] != w5.shape[0]:
        raise ValueError("Expected image channels to be the same as the kernel batches for conv_transpose3d but got %s and %s"
                         % (tuple(x5.shape), tuple(w5.shape)))
    if any(o3pad[i] < 0 or o3pad[i] >= s3[i] for i in range(3)):
        raise ValueError("conv_transpose3d: output_padding must be at least 0 and smaller than the stride")
    k3 = tuple(w5.shape[-3:])
    out3 = tuple((x5.shape[2 + i] - 1) * s3[i] - 2 * p3[i] + d3[i] * (k3[i] - 1) + 1 + o3pad[i] for i in range(3))
    cout = w5.shape[1] * groups
    return k3, out3, cout


def conv_transpose3d(x, w, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    """functional::conv_transpose3d: x [B, Cin, Di, Hi, Wi], w [Cin, Cout/groups, kd, kh, kw] -> [B, Cout, Do, Ho, Wo],
    evaluated as the image gradient of the convolution with the same kernel."""
    x5, w5, s3, p3, d3 = _conv3d_setup(x, w, stride, padding, dilation, groups, "conv3d transpose")
    k3, out3, cout = _transpose3_geom(x5, w5, s3, p3, _triple(output_padding), d3, groups)
    bsz, cin = x5.shape[:2]
    geom = _geom3(bsz, cout, out3, cin, groups, k3, s3, p3, d3)
    code = dtype_code(x)
    ws = torch.empty(max(1, lib().ntb200_conv3d_workspace_bytes(code, ctypes.byref(geom))), dtype=torch.uint8, device=x.device)
    out = torch.empty((bsz, cout) + out3, dtype=x.dtype, device=x.device)
    check(lib().ntb200_conv3d_backward_image(code, x5.data_ptr(), w5.data_ptr(), out.data_ptr(), ws.data_ptr(), ctypes.byref(geom),
                                             _stream()))
    return out


def conv_transpose3d_backward(x, w, grad, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    x5, w5, s3, p3, d3 = _conv3d_setup(x, w, stride, padding, dilation, groups, "conv3d transpose")
    _require_cuda(grad)
    k3, out3, cout = _transpose3_geom(x5, w5, s3, p3, _triple(output_padding), d3, groups)
    bsz, cin = x5.shape[:2]
    geom = _geom3(bsz, cout, out3, cin, groups, k3, s3, p3, d3)
    code = dtype_code(x)
    g = grad.contiguous()
    ws = torch.empty(max(1, lib().ntb200_conv3d_workspace_bytes(code, ctypes.byref(geom))), dtype=torch.uint8, device=x.device)
    dx, dw_ = torch.empty_like(x5), torch.empty_like(w5)
    check(lib().ntb200_conv3d(code, g.data_ptr(), w5.data_ptr(), dx.data_ptr(), ws.data_ptr(), ctypes.byref(geom), _stream()))
    check(lib().ntb200_conv3d_backward_kernel(code, g.data_ptr(), x5.data_ptr(), dw_.data_ptr(), ws.data_ptr(), 0,
                                              ctypes.byref(geom), _stream()))
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def _ntuple(v, n):
    t = tuple(v) if isinstance(v, (tuple, list)) else (v,) * n
    if len(t) != n:
        raise ValueError("Error, expected a single value or %d values (one per dimension), got %d" % (n, len(t)))
    return t


def _geomn(dim, bsz, ch, size, cout, groups, k, s, p, d):
    if dim > _lib.ConvNdGeom.MAX_DIMS:
        raise ValueError("convnd: at most %d spatial dimensions (got %d)" % (_lib.ConvNdGeom.MAX_DIMS, dim))
    g = _lib.ConvNdGeom()
    g.dims, g.batch, g.channels, g.cout, g.groups = dim, bsz, ch, cout, groups
    for arr, val in ((g.size, size), (g.kernel, k), (g.stride, s), (g.padding, p), (g.dilation, d)):
        for i in range(dim):
            arr[i] = val[i]
    return g


def _convnd_setup(x, w, dim, stride, padding, dilation, what="conv"):
    _require_cuda(x, w)
    if dim <= 0:
        raise ValueError("Error, cannot do a dynamic ConvND where N < 0 got (N = %d)" % dim)
    if x.dim() < dim + 1:
        raise ValueError("Expected to get a %dD or greater tensor as the input for a %dd convolution, but got %dD" % (dim + 1, dim, x.dim()))
    if w.dim() not in (dim + 1, dim + 2):
        raise ValueError("Expected to get a %dD or %dD tensor as the kernel for a %dd convolution, but got %dD" % (dim + 1, dim + 2, dim, w.dim()))
    if x.dtype != w.dtype:
        raise ValueError("Expected both kernel and image to have the same dtype for %s%dd but got %s and %s" % (what, dim, w.dtype, x.dtype))
    wn = (w.unsqueeze(0) if w.dim() == dim + 1 else w).contiguous()
    xn = (x.unsqueeze(0) if x.dim() == dim + 1 else x.reshape((-1,) + tuple(x.shape[-(dim + 1):]))).contiguous()
    s, p, d = _ntuple(stride, dim), _ntuple(padding, dim), _ntuple(dilation, dim)
    if min(s) < 1:
        raise ValueError("Conv%dD stride cannot be less than 1" % dim)
    if min(d) < 1:
        raise ValueError("Conv%dD dilation cannot be less than 1" % dim)
    if min(p) < 0:
        raise ValueError("Conv%dD padding cannot be less than 0" % dim)
    return xn, wn, s, p, d


def _outn(size, k, s, p, d):
    return tuple((size[i] + 2 * p[i] - d[i] * (k[i] - 1) - 1) // s[i] + 1 for i in range(len(size)))


def _workspace_nd(code, geom, device):
    return torch.empty(max(1, lib().ntb200_convnd_workspace_bytes(code, ctypes.byref(geom))), dtype=torch.uint8, device=device)


def unfoldnd(x, dim, kernel_size, dilation=1, padding=0, stride=1):
    """functional::unfoldnd with transpose_out (colim_transform.h:106; cpu/unfoldnd.cpp): x [B, C, size...] ->
    col [B, C*prod(kernel), prod(out)], rows ordered (c, k_0 .. k_{N-1}), columns (o_0 .. o_{N-1})."""
    _require_cuda(x)
    xn = x.contiguous()
    k, s, p, d = _ntuple(kernel_size, dim), _ntuple(stride, dim), _ntuple(padding, dim), _ntuple(dilation, dim)
    bsz, ch = xn.shape[:2]
    size = tuple(xn.shape[2:])
    on = _outn(size, k, s, p, d)
    if min(on) <= 0:
        raise ValueError("unfoldnd: calculated output size %s must be at least one" % (on,))
    geom = _geomn(dim, bsz, ch, size, 1, 1, k, s, p, d)
    taps = 1
    for v in k:
        taps *= v
    L = 1
    for v in on:
        L *= v
    col = torch.empty((bsz, ch * taps, L), dtype=x.dtype, device=x.device)
    check(lib().ntb200_im2colnd(dtype_code(x), xn.data_ptr(), col.data_ptr(), ctypes.byref(geom), _stream()))
    return col


def unfoldnd_backward(dcol, dim, output_size, kernel_size, dilation=1, padding=0, stride=1):
    """functional::unfoldnd_backward (colim_transform.h:112): the adjoint of unfoldnd -> [B, C, size...]."""
    _require_cuda(dcol)
    k, s, p, d = _ntuple(kernel_size, dim), _ntuple(stride, dim), _ntuple(padding, dim), _ntuple(dilation, dim)
    size = _ntuple(output_size, dim)
    taps = 1
    for v in k:
        taps *= v
    bsz, ch = dcol.shape[0], dcol.shape[1] // taps
    geom = _geomn(dim, bsz, ch, size, 1, 1, k, s, p, d)
    im = torch.empty((bsz, ch) + size, dtype=dcol.dtype, device=dcol.device)
    check(lib().ntb200_col2imnd(dtype_code(dcol), dcol.contiguous().data_ptr(), im.data_ptr(), ctypes.byref(geom), _stream()))
    return im


def convnd(x, w, dim, stride=1, padding=0, dilation=1, groups=1):
    """functional::convnd (conv.cpp:177-262) -> [B, Cout, out_0 .. out_{N-1}]; w is [Cout, C/groups, k_0 .. k_{N-1}]."""
    xn, wn, s, p, d = _convnd_setup(x, w, dim, stride, padding, dilation)
    bsz, ch = xn.shape[:2]
    cout, k = wn.shape[0], tuple(wn.shape[2:])
    if groups < 1 or ch % groups:
        raise ValueError("Expected image channels to be divisible by groups in Conv%dd but got %d %% %d != 0" % (dim, ch, groups))
    if wn.shape[1] * groups != ch:
        raise ValueError("Expected kernel rows times groups to be equal to rows of image Conv%dd but got %d * %d != %d"
                         % (dim, wn.shape[1], groups, ch))
    size = tuple(xn.shape[2:])
    on = _outn(size, k, s, p, d)
    if min(on) <= 0:
        raise ValueError("conv%dd: calculated output size %s must be at least one" % (dim, on))
    geom = _geomn(dim, bsz, ch, size, cout, groups, k, s, p, d)
    code = dtype_code(x)
    ws = _workspace_nd(code, geom, x.device)
    out = torch.empty((bsz, cout) + on, dtype=x.dtype, device=x.device)
    check(lib().ntb200_convnd(code, xn.data_ptr(), wn.data_ptr(), out.data_ptr(), ws.data_ptr(), ctypes.byref(geom), _stream()))
    return out


def convnd_backward(x, w, grad, dim, stride=1, padding=0, dilation=1, groups=1):
    """conv_dimage / conv_dkernel for any dimension (conv.cpp:378-410, 501-560) -> (d_image, d_kernel)."""
    xn, wn, s, p, d = _convnd_setup(x, w, dim, stride, padding, dilation)
    _require_cuda(grad)
    bsz, ch = xn.shape[:2]
    cout, k = wn.shape[0], tuple(wn.shape[2:])
    geom = _geomn(dim, bsz, ch, tuple(xn.shape[2:]), cout, groups, k, s, p, d)
    code = dtype_code(x)
    g = grad.contiguous()
    ws = _workspace_nd(code, geom, x.device)
    dx, dw_ = torch.empty_like(xn), torch.empty_like(wn)
    check(lib().ntb200_convnd_backward_image(code, g.data_ptr(), wn.data_ptr(), dx.data_ptr(), ws.data_ptr(), ctypes.byref(geom),
                                             _stream()))
    check(lib().ntb200_convnd_backward_kernel(code, xn.data_ptr(), g.data_ptr(), dw_.data_ptr(), ws.data_ptr(), 0,
                                              ctypes.byref(geom), _stream()))
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def _transposen_geom(xn, wn, dim, s, p, opad, d, groups):
    if xn.shape[1] != wn.shape[0]:
        raise ValueError("Expected image channels to be the same as the kernel batches for conv_transpose%dd but got %s and %s"
                         % (dim, tuple(xn.shape), tuple(wn.shape)))
    if any(opad[i] < 0 or opad[i] >= s[i] for i in range(dim)):
        raise ValueError("conv_transpose%dd: output_padding must be at least 0 and smaller than the stride" % dim)
    k = tuple(wn.shape[2:])
    outn = tuple((xn.shape[2 + i] - 1) * s[i] - 2 * p[i] + d[i] * (k[i] - 1) + 1 + opad[i] for i in range(dim))
    return k, outn, wn.shape[1] * groups


def conv_transposend(x, w, dim, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    """functional::conv_transposend (conv.cpp:747-860): x [B, Cin, size...], w [Cin, Cout/groups, k...] ->
    [B, Cout, out...], evaluated as the image gradient of the convolution with the same kernel."""
    xn, wn, s, p, d = _convnd_setup(x, w, dim, stride, padding, dilation, "conv transpose")
    k, outn, cout = _transposen_geom(xn, wn, dim, s, p, _ntuple(output_padding, dim), d, groups)
    bsz, cin = xn.shape[:2]
    geom = _geomn(dim, bsz, cout, outn, cin, groups, k, s, p, d)
    code = dtype_code(x)
    ws = _workspace_nd(code, geom, x.device)
    out = torch.empty((bsz, cout) + outn, dtype=x.dtype, device=x.device)
    check(lib().ntb200_convnd_backward_image(code, xn.data_ptr(), wn.data_ptr(), out.data_ptr(), ws.data_ptr(), ctypes.byref(geom),
                                             _stream()))
    return out


def conv_transposend_backward(x, w, grad, dim, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    xn, wn, s, p, d = _convnd_setup(x, w, dim, stride, padding, dilation, "conv transpose")
    _require_cuda(grad)
    k, outn, cout = _transposen_geom(xn, wn, dim, s, p, _ntuple(output_padding, dim), d, groups)
    bsz, cin = xn.shape[:2]
    geom = _geomn(dim, bsz, cout, outn, cin, groups, k, s, p, d)
    code = dtype_code(x)
    g = grad.contiguous()
    ws = _workspace_nd(code, geom, x.device)
    dx, dw_ = torch.empty_like(xn), torch.empty_like(wn)
    check(lib().ntb200_convnd(code, g.data_ptr(), wn.data_ptr(), dx.data_ptr(), ws.data_ptr(), ctypes.byref(geom), _stream()))
    check(lib().ntb200_convnd_backward_kernel(code, g.data_ptr(), xn.data_ptr(), dw_.data_ptr(), ws.data_ptr(), 0,
                                              ctypes.byref(geom), _stream()))
    return dx.reshape(x.shape), dw_.reshape(w.shape)


def relu(x):
    _require_cuda(x)
    x = x.contiguous()
    y = torch.empty_like(x)
    check(lib().ntb200_relu(dtype_code(x), x.data_ptr(), y.data_ptr(), x.numel(), _stream()))
    return y


def relu_backward(x, grad_out):
    x, grad_out = x.contiguous(), grad_out.contiguous()
    gi = torch.empty_like(grad_out)
    check(lib().ntb200_relu_backward(dtype_code(x), x.data_ptr(), grad_out.data_ptr(), gi.data_ptr(), x.numel(),
                                     _stream()))
    return gi


def bias_add_channels(x, bias):
    """layers::Conv2D's `outp + Bias` (Conv2D.cpp:43): x [B, C, ...] += bias [C] (or [C, 1, 1]) in place."""
    _require_cuda(x, bias)
    if x.dim() < 2 or not x.is_contiguous() or bias.numel() != x.shape[1] or bias.dtype != x.dtype:
        raise ValueError("bias_add_channels: x must be contiguous [B, C, ...] and bias must hold C values of x's dtype")
    inner = x.numel() // max(1, x.shape[0] * x.shape[1])
    b = bias.contiguous()
    check(lib().ntb200_bias_add_channels(dtype_code(x), x.data_ptr(), b.data_ptr(), x.shape[0], x.shape[1], inner, _stream()))
    return x


def sum_channels(grad):
    """Bias gradient of layers::Conv2D: sum of grad [B, C, ...] over the batch and the trailing dims -> [C]."""
    _require_cuda(grad)
    if grad.dim() < 2:
        raise ValueError("sum_channels: expected [B, C, ...]")
    g = grad.contiguous()
    out = torch.empty((g.shape[1],), dtype=g.dtype, device=g.device)
    inner = g.numel() // max(1, g.shape[0] * g.shape[1])
    check(lib().ntb200_sum_channels(dtype_code(g), g.data_ptr(), out.data_ptr(), g.shape[0], g.shape[1], inner, _stream()))
    return out


def sgd_step(param, grad, lr=0.01):
    """optimizers::SGD::step for one parameter (Optimizers.cpp:8-17): param -= clip(grad, -10, 10) * lr, in place."""
    _require_cuda(param, grad)
    if not param.is_contiguous():
        raise ValueError("sgd_step: the parameter must be contiguous (it is updated in place)")
    g = grad.contiguous()
    check(lib().ntb200_sgd_step(dtype_code(param), param.data_ptr(), g.data_ptr(), param.numel(), float(lr), _stream()))
    return param


def adam_step(param, grad, m, v, lr=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, t=0):
    """optimizers::Adam::step for one parameter (Optimizers.cpp:68-98), with the reference's own update rule and its
    step counter `t` (which the reference leaves at 0); param, m and v are updated in place."""
    _require_cuda(param, grad, m, v)
    for name, x in (("param", param), ("m", m), ("v", v)):
        if not x.is_contiguous():
            raise ValueError("adam_step: %s must be contiguous (it is updated in place)" % name)
    g = grad.contiguous()
    check(lib().ntb200_adam_step(dtype_code(param), param.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                 param.numel(), float(lr), float(beta1), float(beta2), float(epsilon), int(t), _stream()))
    return param


def mse(out, target, want_grad=True):
    """loss::MSE -> (loss as a 1-element float32 device tensor, dx or None)."""
    out, target = out.contiguous(), target.contiguous()
    loss = torch.empty(1, dtype=torch.float32, device=out.device)
    grad = torch.empty_like(out) if want_grad else None
    check(lib().ntb200_mse(dtype_code(out), out.data_ptr(), target.data_ptr(), grad.data_ptr() if want_grad else None,
                           loss.data_ptr(), out.numel(), _stream()))
    return loss, grad



def mse_grad_block(out_block, target_block, numel_total):
    """The gradient loss::MSE gives for a [rows, cols] block (views with unit column stride) of a matrix of
    `numel_total` elements: the values mse() writes at those positions, as a contiguous [rows, cols] tensor."""
    _require_cuda(out_block, target_block)
    if out_block.dim() != 2 or out_block.shape != target_block.shape or out_block.stride(1) != 1 or target_block.stride(1) != 1:
        raise ValueError("mse_grad_block takes two [rows, cols] blocks of the same shape with unit column stride")
    if out_block.dtype != target_block.dtype:
        raise ValueError("Expected both tensors to have the same dtype for MSE")
    rows, cols = out_block.shape
    grad = torch.empty((rows, cols), dtype=out_block.dtype, device=out_block.device)
    check(lib().ntb200_mse_grad_block(dtype_code(out_block), out_block.data_ptr(), out_block.stride(0), target_block.data_ptr(),
                                      target_block.stride(0), grad.data_ptr(), cols, rows, cols, int(numel_total), _stream()))
    return grad

def column_sum(grad):
    g2 = grad.reshape(-1, grad.shape[-1]).contiguous()
    out = torch.empty(g2.shape[1], dtype=grad.dtype, device=grad.device)
    check(lib().ntb200_column_sum(dtype_code(g2), g2.data_ptr(), out.data_ptr(), g2.shape[0], g2.shape[1], _stream()))
    return out


def matmult_backward(a, b, grad, transpose_a=False, transpose_b=False):
    """The two transposed GEMMs of nn/functional/matmult.cpp:37-63 (flags only, nothing is materialised)."""
    if transpose_a:
        da = matmult(b, grad, transpose_b, True)
    else:
        da = matmult(grad, b, False, not transpose_b)
    if transpose_b:
        db = matmult(grad, a, True, transpose_a)
    else:
        db = matmult(a, grad, not transpose_a, False)
    return da, db


def matmult_host(a, b, c, transpose_a=False, transpose_b=False, accumulate=True):
    """The raw nt_matmult / nt_matmult_batch contract on HOST arrays (torch CPU tensors or numpy arrays, ideally
    pinned): c += op(a).op(b) (or c = op(a).op(b) with accumulate=False), staged through the device by the
    library.  a, b, c are 2-D or 3-D and contiguous."""
    import numpy as np

    np_codes = {"float32": _lib.F32, "float16": _lib.F16, "int8": _lib.I8, "int16": _lib.I16, "int32": _lib.I32,
                "int64": _lib.I64, "float64": _lib.F64, "uint8": _lib.U8, "uint16": _lib.U16, "uint32": _lib.U32}

    def info(t):
        if isinstance(t, torch.Tensor):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("matmult_host expects contiguous host tensors")
            return t.data_ptr(), tuple(t.shape), dtype_code(t)
        if not isinstance(t, np.ndarray) or not t.flags.c_contiguous:
            raise ValueError("matmult_host expects contiguous host arrays")
        return t.ctypes.data, t.shape, np_codes[t.dtype.name]

    pa, sa, ca = info(a)
    pb, sb, cb = info(b)
    pc, sc, cc = info(c)
    if not (ca == cb == cc):
        raise ValueError("matmult_host operands must share a dtype")
    batches = sa[0] if len(sa) == 3 else 1
    am, ak = (sa[-1], sa[-2]) if transpose_a else (sa[-2], sa[-1])
    bk, bn = (sb[-1], sb[-2]) if transpose_b else (sb[-2], sb[-1])
    check(lib().ntb200_matmult_host(ca, pa, pb, pc, batches, am, ak, bk, bn, int(transpose_a), int(transpose_b),
                                    int(bool(accumulate))))
    return c
