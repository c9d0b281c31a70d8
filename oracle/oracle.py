"""TEST INFRASTRUCTURE ONLY -- numpy front end of the CPU oracle.

Imported by tests/, by the smoke test and by the benchmark's CPU-baseline leg; never by the package.
The arithmetic lives in oracle.cpp (built by `make -C oracle`); this file restates the reference's
host-side shape rules on numpy arrays, each function citing the reference file it follows (paths
relative to the reference project root):

  matmult / batched matmult   nt/functional/cpu/matmult_cpu.cpp:51-121,654-750,863-1005
  linear                      nt/functional/cpu/matmult_cpu.cpp:1624-1714
  unfold2d / conv2d           nt/functional/tensor_files/colim_transform.cpp:565-588, conv.cpp:69-96
  conv backward               nt/functional/tensor_files/conv.cpp:318-346,444-471
  matmult / linear backward   nt/nn/functional/matmult.cpp:37-63,253-273
  relu (clamp) / MSE          nt/nn/functional/min_max.cpp:40-63, nt/nn/Loss.cpp:49-55

Parity status: Float32 is pinned by the reference's committed golden vectors (tests/golden/);
Float16 / integer / BFloat16 are "parity unpinned" by tests and follow the source semantics.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

# dtype codes shared with include/ntb200.h
F32, F16, BF16, I8, I16, I32, I64, F64, U8, U16, U32 = range(11)

_NP_TO_CODE = {
    np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.int8): I8, np.dtype(np.int16): I16,
    np.dtype(np.int32): I32, np.dtype(np.int64): I64, np.dtype(np.float64): F64, np.dtype(np.uint8): U8,
    np.dtype(np.uint16): U16, np.dtype(np.uint32): U32,
}


def build(force=False):
    """Compile liboracle.so with the committed Makefile (no-op when it is already there)."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.check_call(["make", "-C", _HERE] + (["-B"] if force else []))
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        _lib.oracle_matmult.argtypes = [ci, vp, vp, vp, i64, i64, i64, i64, ci, ci, ci]
        _lib.oracle_matmult.restype = ci
        _lib.oracle_im2col.argtypes = [ci, vp, vp] + [i64] * 12
        _lib.oracle_im2col.restype = ci
        _lib.oracle_col2im_f32.argtypes = [vp, vp] + [i64] * 12
        _lib.oracle_col2im_f32.restype = ci
        _lib.oracle_hardware_threads.restype = ci
    return _lib


def hardware_threads():
    return int(lib().oracle_hardware_threads())


def default_threads():
    """The reference caps its GEMM at 21 TBB threads (nt_matmult_macros.h:42)."""
    return max(1, min(21, hardware_threads()))


def bf16_round(x32):
    """float32 -> bfloat16 bit pattern (uint16), round to nearest even."""
    u = np.ascontiguousarray(x32, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_widen(bits):
    """bfloat16 bit pattern (uint16) -> float32, exact."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


F16_TILE8 = 100   # one lane of a Complex32 product: Float16 rounded every 8 k-steps


def _code(arr, bf16):
    if bf16 == "c32-lane":
        assert arr.dtype == np.float16
        return F16_TILE8
    if bf16:
        assert arr.dtype == np.uint16, "bf16 operands are passed as uint16 bit patterns"
        return BF16
    return _NP_TO_CODE[arr.dtype]


def matmult_complex32(a, b, transpose_a=False, transpose_b=False, threads=None):
    """Complex32 matmult as the reference computes it.  Operands are float16 arrays whose last axis holds (re, im).
    The reference's traits for complex_32 are the float lane operations on the widened interleaved halves
    (nt/mp/simde_traits/simde_traits_avx2.h:1270-1400), so real parts meet real parts and imaginary parts imaginary
    parts, each an fp32 chain rounded to Float16 at the type's K-tile edges, every 8 k-steps."""
    assert a.dtype == np.float16 and b.dtype == np.float16 and a.shape[-1] == 2 and b.shape[-1] == 2
    re = matmult(np.ascontiguousarray(a[..., 0]), np.ascontiguousarray(b[..., 0]), transpose_a, transpose_b, "c32-lane", threads)
    im = matmult(np.ascontiguousarray(a[..., 1]), np.ascontiguousarray(b[..., 1]), transpose_a, transpose_b, "c32-lane", threads)
    return np.stack([re, im], axis=-1)


def matmult_into(a, b, c, transpose_a=False, transpose_b=False, bf16=False, threads=None):
    """C += op(A).op(B) on 2-D contiguous arrays: the raw nt_matmult<T> contract."""
    assert a.ndim == 2 and b.ndim == 2 and c.ndim == 2
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert c.flags.c_contiguous and a.dtype == b.dtype == c.dtype
    m, k = (a.shape[1], a.shape[0]) if transpose_a else a.shape
    k2, n = (b.shape[1], b.shape[0]) if transpose_b else b.shape
    if k != k2:
        raise ValueError(f"matmult shape mismatch {a.shape} {b.shape} ta={transpose_a} tb={transpose_b}")
    assert c.shape == (m, n)
    rc = lib().oracle_matmult(_code(a, bf16), a.ctypes.data, b.ctypes.data, c.ctypes.data, m, k, k2, n,
                              int(transpose_a), int(transpose_b), threads or default_threads())
    if rc:
        raise RuntimeError(f"oracle_matmult failed rc={rc}")
    return c


_ref_lib = None


def reference_lib():
    """The reference's own matmult kernel compiled from its sources (oracle/build_ref.py), or None when neither the
    reference tree nor a prebuilt oracle/_ref/libntref.so is present."""
    global _ref_lib
    if _ref_lib is None:
        from . import build_ref
        path = build_ref.build()
        if path is None:
            return None
        handle = ctypes.CDLL(path)
        handle.ntref_matmult.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 4 + [ctypes.c_int] * 2
        _ref_lib = handle
    return _ref_lib


def reference_matmult(a, b, transpose_a=False, transpose_b=False):
    """C = op(A).op(B) by the REFERENCE's compiled nt_matmult<T> (2-D or batched, one item after the other as
    nt_matmult_batch does), from a zero-filled C as functional::matmult calls it.  Uses the host threads the
    reference would (up to 21).  No BFloat16: the reference has no such dtype."""
    L = reference_lib()
    if L is None:
        raise RuntimeError("the reference's kernel is not available here (no reference tree, no prebuilt library)")
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    batched = a.ndim == 3
    a3, b3 = (a, b) if batched else (a[None], b[None])
    m, k = (a3.shape[2], a3.shape[1]) if transpose_a else a3.shape[1:]
    k2, n = (b3.shape[2], b3.shape[1]) if transpose_b else b3.shape[1:]
    assert k == k2 and a3.shape[0] == b3.shape[0]
    c = np.zeros((a3.shape[0], m, n), dtype=a.dtype)
    code = _code(a, False)
    for i in range(a3.shape[0]):
        rc = L.ntref_matmult(code, a3[i].ctypes.data, b3[i].ctypes.data, c[i].ctypes.data, m, k, k2, n, int(transpose_a), int(transpose_b))
        if rc:
            raise RuntimeError("the reference kernel has no instantiation for %s" % a.dtype)
    return c if batched else c[0]


def matmult(a, b, transpose_a=False, transpose_b=False, bf16=False, threads=None):
    """functional::matmult: 2-D x 2-D, N-D x N-D with equal leading dims, or one operand of lower
    rank repeated over the other's batch (matmult_cpu.cpp:863-1005).  Result starts from zeros."""
    if a.ndim < 2 or b.ndim < 2:
        raise ValueError("matmult needs tensors of at least 2 dims")
    if a.dtype != b.dtype:
        raise ValueError("matmult operands must share a dtype")
    if np.iscomplexobj(a):
        # Complex64 / Complex128: the SIMD traits of these types are the float / double operations on the interleaved
        # (re, im) lanes (nt/mp/simde_traits/simde_traits_avx2.h:915-1000, 1029-1110: broadcast = set1 of the pair,
        # fmadd = _mm256_fmadd_ps / _pd), so the microkernel multiplies re with re and im with im: two independent
        # real matmults, not the mathematical complex product.
        out_re = matmult(np.ascontiguousarray(a.real), np.ascontiguousarray(b.real), transpose_a, transpose_b, False, threads)
        out_im = matmult(np.ascontiguousarray(a.imag), np.ascontiguousarray(b.imag), transpose_a, transpose_b, False, threads)
        out = np.empty(out_re.shape, dtype=a.dtype)
        out.real, out.imag = out_re, out_im
        return out
    am, ak = (a.shape[-1], a.shape[-2]) if transpose_a else a.shape[-2:]
    bk, bn = (b.shape[-1], b.shape[-2]) if transpose_b else b.shape[-2:]
    if ak != bk:
        raise ValueError(f"matmult shape mismatch {a.shape} {b.shape}")
    lead_a, lead_b = a.shape[:-2], b.shape[:-2]
    if len(lead_a) >= len(lead_b):
        lead = lead_a
        if lead_b and lead_a[len(lead_a) - len(lead_b):] != lead_b:
            raise ValueError("batch dims must match on the shared suffix")
    else:
        lead = lead_b
        if lead_a and lead_b[len(lead_b) - len(lead_a):] != lead_a:
            raise ValueError("batch dims must match on the shared suffix")
    nb = int(np.prod(lead)) if lead else 1
    a3 = np.ascontiguousarray(np.broadcast_to(a, lead + a.shape[-2:])).reshape((nb,) + a.shape[-2:])
    b3 = np.ascontiguousarray(np.broadcast_to(b, lead + b.shape[-2:])).reshape((nb,) + b.shape[-2:])
    out = np.zeros((nb, am, bn), dtype=a.dtype)
    for i in range(nb):
        matmult_into(a3[i], b3[i], out[i], transpose_a, transpose_b, bf16, threads)
    return out.reshape(lead + (am, bn))


def linear(x, w, bias=None, transpose_a=False, transpose_b=False, bf16=False, threads=None):
    """functional::linear: C starts as the broadcast bias, then C += op(x).op(w)."""
    if bias is None:
        return matmult(x, w, transpose_a, transpose_b, bf16, threads)
    m = x.shape[-1] if transpose_a else x.shape[-2]
    n = w.shape[-2] if transpose_b else w.shape[-1]
    lead = x.shape[:-2] if x.ndim >= w.ndim else w.shape[:-2]
    nb = int(np.prod(lead)) if lead else 1
    out = np.ascontiguousarray(np.broadcast_to(bias, lead + (m, n))).reshape(nb, m, n).copy()
    x3 = np.ascontiguousarray(np.broadcast_to(x, lead + x.shape[-2:])).reshape((nb,) + x.shape[-2:])
    w3 = np.ascontiguousarray(np.broadcast_to(w, lead + w.shape[-2:])).reshape((nb,) + w.shape[-2:])
    for i in range(nb):
        matmult_into(x3[i], w3[i], out[i], transpose_a, transpose_b, bf16, threads)
    return out.reshape(lead + (m, n))


def _pair(v):
    return (int(v), int(v)) if np.isscalar(v) else (int(v[0]), int(v[1]))


def conv_out_size(size, k, s, p, d):
    return (size + 2 * p - d * (k - 1) - 1) // s + 1


def unfold2d(x, kernel_size, dilation=1, padding=0, stride=1, bf16=False):
    """functional::unfold2d(..., transpose_out=true): [B, C*kh*kw, L]."""
    kh, kw = _pair(kernel_size)
    dh, dw = _pair(dilation)
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    x4 = np.ascontiguousarray(x.reshape((-1,) + x.shape[-3:]))
    bsz, ch, h, w = x4.shape
    hc, wc = conv_out_size(h, kh, sh, ph, dh), conv_out_size(w, kw, sw, pw, dw)
    col = np.zeros((bsz, ch * kh * kw, hc * wc), dtype=x.dtype)
    rc = lib().oracle_im2col(_code(x4, bf16), x4.ctypes.data, col.ctypes.data, bsz, ch, h, w, kh, kw, sh, sw, ph, pw,
                             dh, dw)
    assert rc == 0
    return col


def unfold2d_backward(dcol, out_hw, kernel_size, dilation=1, padding=0, stride=1):
    kh, kw = _pair(kernel_size)
    dh, dw = _pair(dilation)
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    h, w = out_hw
    dcol = np.ascontiguousarray(dcol, dtype=np.float32)
    bsz = dcol.shape[0]
    ch = dcol.shape[1] // (kh * kw)
    im = np.zeros((bsz, ch, h, w), dtype=np.float32)
    rc = lib().oracle_col2im_f32(dcol.ctypes.data, im.ctypes.data, bsz, ch, h, w, kh, kw, sh, sw, ph, pw, dh, dw)
    assert rc == 0
    return im


def conv2d(x, w, stride=1, padding=0, dilation=1, bf16=False, threads=None, groups=1):
    """functional::conv2d: matmult(col, w2d, true, true) -> [B, L, Cout], then the row/col swap and the view to
    [B, Cout, Ho, Wo] (conv.cpp:94-95); with groups the column matrix is split into `groups` row blocks and the
    kernel into `groups` filter blocks, multiplied pairwise and interleaved back (conv.cpp:97-118)."""
    kh, kw = w.shape[-2:]
    dh, dw = _pair(dilation)
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    x4 = x.reshape((-1,) + x.shape[-3:])
    ho = conv_out_size(x4.shape[-2], kh, sh, ph, dh)
    wo = conv_out_size(x4.shape[-1], kw, sw, pw, dw)
    col = unfold2d(x4, (kh, kw), dilation, padding, stride, bf16)
    cout = w.shape[0]
    ckg, coutg = col.shape[1] // groups, cout // groups
    outs = []
    for g in range(groups):
        col_g = np.ascontiguousarray(col[:, g * ckg:(g + 1) * ckg])
        w2d = np.ascontiguousarray(w[g * coutg:(g + 1) * coutg].reshape(coutg, -1))
        out = matmult(col_g, w2d, True, True, bf16, threads)        # [B, L, Cout/groups]
        outs.append(out.transpose(0, 2, 1))
    return np.ascontiguousarray(np.concatenate(outs, axis=1)).reshape(x4.shape[0], cout, ho, wo)


def conv2d_backward(x, w, grad, stride=1, padding=0, dilation=1, threads=None, groups=1):
    """conv_dimage (conv.cpp:318-346) and conv_dkernel (conv.cpp:444-471), Float32, group by group."""
    kh, kw = w.shape[-2:]
    x4 = x.reshape((-1,) + x.shape[-3:])
    bsz, cout = x4.shape[0], w.shape[0]
    col = unfold2d(x4, (kh, kw), dilation, padding, stride)
    g3 = np.ascontiguousarray(grad.reshape(bsz, cout, -1))
    ckg, coutg = col.shape[1] // groups, cout // groups
    dcol = np.empty_like(col)
    dw = np.empty((cout, ckg), dtype=np.float32)
    for g in range(groups):
        w2d = np.ascontiguousarray(w[g * coutg:(g + 1) * coutg].reshape(coutg, -1))
        gg = np.ascontiguousarray(g3[:, g * coutg:(g + 1) * coutg])
        dcol[:, g * ckg:(g + 1) * ckg] = matmult(w2d, gg, True, False, threads=threads)      # [B, ckg, L]
        col_g = np.ascontiguousarray(col[:, g * ckg:(g + 1) * ckg])
        dw[g * coutg:(g + 1) * coutg] = matmult(gg, col_g, False, True, threads=threads).sum(axis=0, dtype=np.float32)
    dx = unfold2d_backward(dcol, x4.shape[-2:], (kh, kw), dilation, padding, stride).reshape(x.shape)
    return dx, dw.reshape(w.shape)


def conv_transpose2d(x, w, stride=1, padding=0, output_padding=0, dilation=1, groups=1, threads=None):
    """functional::conv_transpose2d (conv.cpp:614-672): the input is dilated by the stride (zeros between its
    elements), padded at the end by output_padding, and convolved with stride 1 and padding d*(k-1) - p by the
    kernel with its two channel axes swapped (within each group) and both spatial axes flipped."""
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    oh, ow = _pair(output_padding)
    dh, dw = _pair(dilation)
    x4 = x.reshape((-1,) + x.shape[-3:])
    bsz, cin, hi, wi = x4.shape
    kh, kw = w.shape[-2:]
    xd = np.zeros((bsz, cin, (hi - 1) * sh + 1 + oh, (wi - 1) * sw + 1 + ow), dtype=x.dtype)
    xd[:, :, :(hi - 1) * sh + 1:sh, :(wi - 1) * sw + 1:sw] = x4
    cing, coutg = cin // groups, w.shape[1]
    wf = np.empty((coutg * groups, cing, kh, kw), dtype=w.dtype)
    for g in range(groups):     # w.transpose(0, 1).flip({-1, -2}), group by group
        blk = w[g * cing:(g + 1) * cing]                                    # [cin/g, cout/g, kh, kw]
        wf[g * coutg:(g + 1) * coutg] = blk.transpose(1, 0, 2, 3)[:, :, ::-1, ::-1]
    return conv2d(xd, np.ascontiguousarray(wf), 1, (dh * (kh - 1) - ph, dw * (kw - 1) - pw), (dh, dw), threads=threads,
                  groups=groups)


def conv_transpose2d_backward(x, w, grad, stride=1, padding=0, output_padding=0, dilation=1, groups=1, threads=None):
    """Gradients of conv_transpose2d: it is the image-gradient operator of the convolution with the same kernel,
    so d_x is that convolution applied to grad, and d_w is its kernel gradient with grad as the image and x as
    the gradient (nn/functional/conv.cpp, conv_transpose2d backward)."""
    x4 = x.reshape((-1,) + x.shape[-3:])
    g4 = grad.reshape((x4.shape[0], -1) + grad.shape[-2:])
    dx = conv2d(g4, w, stride, padding, dilation, threads=threads, groups=groups).reshape(x.shape)
    _, dw = conv2d_backward(g4, w, x4, stride, padding, dilation, threads=threads, groups=groups)
    return dx, dw


def _triple(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v, v)


def unfold3d(x, kernel_size, dilation=1, padding=0, stride=1):
    """unfold3d (colim_transform.cpp:661-696, cpu/unfold3d.cpp): col[b][((c*kd+kz)*kh+ky)*kw+kx][(z*Ho+y)*Wo+x] =
    x[b][c][z*sd-pd+kz*dd][y*sh-ph+ky*dh][x*sw-pw+kx*dw], zero outside the image."""
    kd, kh, kw = _triple(kernel_size)
    dd, dh, dw = _triple(dilation)
    pd, ph, pw = _triple(padding)
    sd, sh, sw = _triple(stride)
    b, c, D, H, W = x.shape
    od, oh, ow = conv_out_size(D, kd, sd, pd, dd), conv_out_size(H, kh, sh, ph, dh), conv_out_size(W, kw, sw, pw, dw)
    xp = np.zeros((b, c, D + 2 * pd, H + 2 * ph, W + 2 * pw), dtype=x.dtype)
    xp[:, :, pd:pd + D, ph:ph + H, pw:pw + W] = x
    col = np.empty((b, c, kd, kh, kw, od, oh, ow), dtype=x.dtype)
    for kz in range(kd):
        for ky in range(kh):
            for kx in range(kw):
                col[:, :, kz, ky, kx] = xp[:, :, kz * dd:kz * dd + (od - 1) * sd + 1:sd, ky * dh:ky * dh + (oh - 1) * sh + 1:sh,
                                           kx * dw:kx * dw + (ow - 1) * sw + 1:sw]
    return col.reshape(b, c * kd * kh * kw, od * oh * ow)


def unfold3d_backward(dcol, out_dhw, kernel_size, dilation=1, padding=0, stride=1):
    """unfold3d_backward (colim_transform.cpp:698-800): the adjoint of unfold3d, accumulated in Float32."""
    kd, kh, kw = _triple(kernel_size)
    dd, dh, dw = _triple(dilation)
    pd, ph, pw = _triple(padding)
    sd, sh, sw = _triple(stride)
    D, H, W = out_dhw
    b = dcol.shape[0]
    c = dcol.shape[1] // (kd * kh * kw)
    od, oh, ow = conv_out_size(D, kd, sd, pd, dd), conv_out_size(H, kh, sh, ph, dh), conv_out_size(W, kw, sw, pw, dw)
    d8 = dcol.reshape(b, c, kd, kh, kw, od, oh, ow).astype(np.float32)
    xp = np.zeros((b, c, D + 2 * pd, H + 2 * ph, W + 2 * pw), dtype=np.float32)
    for kz in range(kd):
        for ky in range(kh):
            for kx in range(kw):
                xp[:, :, kz * dd:kz * dd + (od - 1) * sd + 1:sd, ky * dh:ky * dh + (oh - 1) * sh + 1:sh,
                   kx * dw:kx * dw + (ow - 1) * sw + 1:sw] += d8[:, :, kz, ky, kx]
    return xp[:, :, pd:pd + D, ph:ph + H, pw:pw + W].astype(dcol.dtype)


def conv3d(x, w, stride=1, padding=0, dilation=1, groups=1, threads=None):
    """functional::conv3d (conv.cpp:122-174): unfold3d, then matmult(col, w2d, true, true) and the row/col swap,
    group by group."""
    x5 = x.reshape((-1,) + x.shape[-4:])
    k3 = w.shape[-3:]
    s3, p3, d3 = _triple(stride), _triple(padding), _triple(dilation)
    o3 = tuple(conv_out_size(x5.shape[2 + i], k3[i], s3[i], p3[i], d3[i]) for i in range(3))
    col = unfold3d(x5, k3, d3, p3, s3)
    cout = w.shape[0]
    ckg, coutg = col.shape[1] // groups, cout // groups
    outs = []
    for g in range(groups):
        col_g = np.ascontiguousarray(col[:, g * ckg:(g + 1) * ckg])
        w2d = np.ascontiguousarray(w[g * coutg:(g + 1) * coutg].reshape(coutg, -1))
        outs.append(matmult(col_g, w2d, True, True, threads=threads).transpose(0, 2, 1))
    return np.ascontiguousarray(np.concatenate(outs, axis=1)).reshape((x5.shape[0], cout) + o3)


def conv3d_backward(x, w, grad, stride=1, padding=0, dilation=1, groups=1, threads=None):
    """conv_dimage / conv_dkernel, dim == 3 (conv.cpp:347-376, 472-500), Float32."""
    x5 = x.reshape((-1,) + x.shape[-4:])
    k3 = w.shape[-3:]
    s3, p3, d3 = _triple(stride), _triple(padding), _triple(dilation)
    bsz, cout = x5.shape[0], w.shape[0]
    col = unfold3d(x5, k3, d3, p3, s3)
    g3 = np.ascontiguousarray(grad.reshape(bsz, cout, -1))
    ckg, coutg = col.shape[1] // groups, cout // groups
    dcol = np.empty_like(col)
    dw = np.empty((cout, ckg), dtype=np.float32)
    for g in range(groups):
        w2d = np.ascontiguousarray(w[g * coutg:(g + 1) * coutg].reshape(coutg, -1))
        gg = np.ascontiguousarray(g3[:, g * coutg:(g + 1) * coutg])
        dcol[:, g * ckg:(g + 1) * ckg] = matmult(w2d, gg, True, False, threads=threads)
        col_g = np.ascontiguousarray(col[:, g * ckg:(g + 1) * ckg])
        dw[g * coutg:(g + 1) * coutg] = matmult(gg, col_g, False, True, threads=threads).sum(axis=0, dtype=np.float32)
    dx = unfold3d_backward(dcol, x5.shape[-3:], k3, d3, p3, s3).reshape(x.shape)
    return dx, dw.reshape(w.shape)


def conv_transpose3d(x, w, stride=1, padding=0, output_padding=0, dilation=1, groups=1, threads=None):
    """functional::conv_transpose3d (conv.cpp:674-735): dilate the input by the stride, pad the end by
    output_padding, convolve with stride 1 and padding d*(k-1) - p by the channel-swapped, flipped kernel."""
    s3, p3, o3, d3 = _triple(stride), _triple(padding), _triple(output_padding), _triple(dilation)
    x5 = x.reshape((-1,) + x.shape[-4:])
    bsz, cin = x5.shape[:2]
    k3 = w.shape[-3:]
    ext = tuple((x5.shape[2 + i] - 1) * s3[i] + 1 + o3[i] for i in range(3))
    xd = np.zeros((bsz, cin) + ext, dtype=x.dtype)
    xd[:, :, :(x5.shape[2] - 1) * s3[0] + 1:s3[0], :(x5.shape[3] - 1) * s3[1] + 1:s3[1], :(x5.shape[4] - 1) * s3[2] + 1:s3[2]] = x5
    cing, coutg = cin // groups, w.shape[1]
    wf = np.empty((coutg * groups, cing) + tuple(k3), dtype=w.dtype)
    for g in range(groups):
        blk = w[g * cing:(g + 1) * cing]
        wf[g * coutg:(g + 1) * coutg] = blk.transpose(1, 0, 2, 3, 4)[:, :, ::-1, ::-1, ::-1]
    pad = tuple(d3[i] * (k3[i] - 1) - p3[i] for i in range(3))
    return conv3d(xd, np.ascontiguousarray(wf), 1, pad, d3, groups=groups, threads=threads)


def conv_transpose3d_backward(x, w, grad, stride=1, padding=0, output_padding=0, dilation=1, groups=1, threads=None):
    x5 = x.reshape((-1,) + x.shape[-4:])
    g5 = grad.reshape((x5.shape[0], -1) + grad.shape[-3:])
    dx = conv3d(g5, w, stride, padding, dilation, groups=groups, threads=threads).reshape(x.shape)
    _, dw = conv3d_backward(g5, w, x5, stride, padding, dilation, groups=groups, threads=threads)
    return dx, dw


def _ntuple(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


def unfoldnd(x, dim, kernel_size, dilation=1, padding=0, stride=1):
    """unfoldnd with transpose_out (cpu/unfoldnd.cpp:327-420): col[b][(c, k_0..k_{N-1})][(o_0..o_{N-1})] =
    x[b][c][o_i*s_i - p_i + k_i*d_i ...], zero outside the image; in 1, 2 and 3 dimensions the layouts of
    unfold1d / unfold2d / unfold3d (the reference asserts this in tests/src/col_im_tests.cpp:47-83)."""
    k, d, p, s = _ntuple(kernel_size, dim), _ntuple(dilation, dim), _ntuple(padding, dim), _ntuple(stride, dim)
    b, c = x.shape[:2]
    size = x.shape[2:]
    o = tuple(conv_out_size(size[i], k[i], s[i], p[i], d[i]) for i in range(dim))
    xp = np.zeros((b, c) + tuple(size[i] + 2 * p[i] for i in range(dim)), dtype=x.dtype)
    xp[(slice(None), slice(None)) + tuple(slice(p[i], p[i] + size[i]) for i in range(dim))] = x
    col = np.empty((b, c) + k + o, dtype=x.dtype)
    for tap in np.ndindex(*k):
        src = tuple(slice(tap[i] * d[i], tap[i] * d[i] + (o[i] - 1) * s[i] + 1, s[i]) for i in range(dim))
        col[(slice(None), slice(None)) + tap] = xp[(slice(None), slice(None)) + src]
    return col.reshape(b, c * int(np.prod(k)), int(np.prod(o)))


def unfoldnd_backward(dcol, dim, out_size, kernel_size, dilation=1, padding=0, stride=1):
    """unfoldnd_backward (cpu/unfoldnd_backward.cpp:323-420): the adjoint of unfoldnd, accumulated in Float32."""
    k, d, p, s = _ntuple(kernel_size, dim), _ntuple(dilation, dim), _ntuple(padding, dim), _ntuple(stride, dim)
    size = tuple(out_size)
    b = dcol.shape[0]
    c = dcol.shape[1] // int(np.prod(k))
    o = tuple(conv_out_size(size[i], k[i], s[i], p[i], d[i]) for i in range(dim))
    dn = dcol.reshape((b, c) + k + o).astype(np.float32)
    xp = np.zeros((b, c) + tuple(size[i] + 2 * p[i] for i in range(dim)), dtype=np.float32)
    for tap in np.ndindex(*k):
        dst = tuple(slice(tap[i] * d[i], tap[i] * d[i] + (o[i] - 1) * s[i] + 1, s[i]) for i in range(dim))
        xp[(slice(None), slice(None)) + dst] += dn[(slice(None), slice(None)) + tap]
    return xp[(slice(None), slice(None)) + tuple(slice(p[i], p[i] + size[i]) for i in range(dim))].astype(dcol.dtype)


def convnd(x, w, dim, stride=1, padding=0, dilation=1, groups=1, threads=None):
    """functional::convnd (conv.cpp:177-262): unfoldnd, then matmult(col, w2d, true, true) and the row/col swap,
    group by group."""
    xn = x.reshape((-1,) + x.shape[-(dim + 1):])
    k = tuple(w.shape[-dim:])
    s, p, d = _ntuple(stride, dim), _ntuple(padding, dim), _ntuple(dilation, dim)
    o = tuple(conv_out_size(xn.shape[2 + i], k[i], s[i], p[i], d[i]) for i in range(dim))
    col = unfoldnd(xn, dim, k, d, p, s)
    cout = w.shape[0]
    ckg, coutg = col.shape[1] // groups, cout // groups
    outs = []
    for g in range(groups):
        col_g = np.ascontiguousarray(col[:, g * ckg:(g + 1) * ckg])
        w2d = np.ascontiguousarray(w[g * coutg:(g + 1) * coutg].reshape(coutg, -1))
        outs.append(matmult(col_g, w2d, True, True, threads=threads).transpose(0, 2, 1))
    return np.ascontiguousarray(np.concatenate(outs, axis=1)).reshape((xn.shape[0], cout) + o)


def convnd_backward(x, w, grad, dim, stride=1, padding=0, dilation=1, groups=1, threads=None):
    """conv_dimage / conv_dkernel, general dimension (conv.cpp:378-410, 501-560), Float32."""
    xn = x.reshape((-1,) + x.shape[-(dim + 1):])
    k = tuple(w.shape[-dim:])
    s, p, d = _ntuple(stride, dim), _ntuple(padding, dim), _ntuple(dilation, dim)
    bsz, cout = xn.shape[0], w.shape[0]
    col = unfoldnd(xn, dim, k, d, p, s)
    g3 = np.ascontiguousarray(grad.reshape(bsz, cout, -1))
    ckg, coutg = col.shape[1] // groups, cout // groups
    dcol = np.empty_like(col)
    dw = np.empty((cout, ckg), dtype=np.float32)
    for g in range(groups):
        w2d = np.ascontiguousarray(w[g * coutg:(g + 1) * coutg].reshape(coutg, -1))
        gg = np.ascontiguousarray(g3[:, g * coutg:(g + 1) * coutg])
        dcol[:, g * ckg:(g + 1) * ckg] = matmult(w2d, gg, True, False, threads=threads)
        col_g = np.ascontiguousarray(col[:, g * ckg:(g + 1) * ckg])
        dw[g * coutg:(g + 1) * coutg] = matmult(gg, col_g, False, True, threads=threads).sum(axis=0, dtype=np.float32)
    dx = unfoldnd_backward(dcol, dim, xn.shape[2:], k, d, p, s).reshape(x.shape)
    return dx, dw.reshape(w.shape)


def conv_transposend(x, w, dim, stride=1, padding=0, output_padding=0, dilation=1, groups=1, threads=None):
    """functional::conv_transposend (conv.cpp:747-860): dilate the input by the stride, pad the end by
    output_padding, convolve with stride 1 and padding d*(k-1) - p by the channel-swapped, flipped kernel."""
    s, p, op, d = _ntuple(stride, dim), _ntuple(padding, dim), _ntuple(output_padding, dim), _ntuple(dilation, dim)
    xn = x.reshape((-1,) + x.shape[-(dim + 1):])
    bsz, cin = xn.shape[:2]
    k = tuple(w.shape[-dim:])
    ext = tuple((xn.shape[2 + i] - 1) * s[i] + 1 + op[i] for i in range(dim))
    xd = np.zeros((bsz, cin) + ext, dtype=x.dtype)
    xd[(slice(None), slice(None)) + tuple(slice(0, (xn.shape[2 + i] - 1) * s[i] + 1, s[i]) for i in range(dim))] = xn
    cing, coutg = cin // groups, w.shape[1]
    wf = np.empty((coutg * groups, cing) + k, dtype=w.dtype)
    flip = (slice(None), slice(None)) + (slice(None, None, -1),) * dim
    for g in range(groups):
        blk = w[g * cing:(g + 1) * cing]
        wf[g * coutg:(g + 1) * coutg] = np.swapaxes(blk, 0, 1)[flip]
    pad = tuple(d[i] * (k[i] - 1) - p[i] for i in range(dim))
    return convnd(xd, np.ascontiguousarray(wf), dim, 1, pad, d, groups=groups, threads=threads)


def conv1d(x, w, stride=1, padding=0, dilation=1, groups=1, threads=None):
    """functional::conv1d (conv.cpp:13-67): unfold1d + matmult, i.e. the one-row case of conv2d."""
    x3 = x.reshape((-1,) + x.shape[-2:])
    out = conv2d(x3[:, :, None, :], w[:, :, None, :], (1, stride), (0, padding), (1, dilation), threads=threads, groups=groups)
    return out[:, :, 0, :]


def matmult_backward(a, b, grad, transpose_a=False, transpose_b=False, bf16=False, threads=None):
    """nn/functional/matmult.cpp:37-63: the two transposed GEMMs, flags only."""
    if transpose_a:
        da = matmult(b, grad, transpose_b, True, bf16, threads)
    else:
        da = matmult(grad, b, False, not transpose_b, bf16, threads)
    if transpose_b:
        db = matmult(grad, a, True, transpose_a, bf16, threads)
    else:
        db = matmult(a, grad, not transpose_a, False, bf16, threads)
    return da, db


def relu(x):
    """clamp(x, 0, none) (nn/functional/min_max.cpp:40-63); the mask is where the value changed."""
    y = np.maximum(x, 0)
    return y, (y != x)


def mse(out, target):
    """loss::MSE (nn/Loss.cpp:49-55): loss = sum((o-t)^2)/numel, dx = 2(o-t)/numel."""
    d = out.astype(np.float32) - target.astype(np.float32)
    return float((d * d).sum(dtype=np.float64) / d.size), (2.0 * d / d.size).astype(np.float32)


def rel_fro(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((x - ref).ravel()) / (den if den > 0 else 1.0))


def _typed_ops(dtype, bf16):
    """(round-to-dtype, scalar-in-dtype) for the optimizers.  bf16 values travel as float32 arrays holding bf16
    numbers; every operation is done in float32 and rounded to bf16, which is how the device computes them."""
    if bf16:
        rnd = lambda x: bf16_widen(bf16_round(np.asarray(x, dtype=np.float32)))
        return rnd, (lambda s: rnd(np.float32(s))[()])
    return (lambda x: np.asarray(x).astype(dtype)), dtype.type


def _clamp10(x, c):
    """std::clamp as clamp_ applies it (nt/functional/cpu/min_max.cpp:66-101): a NaN stays a NaN."""
    return np.where(x < c(-10), c(-10), np.where(c(10) < x, c(10), x))


def sgd_step(param, grad, lr=0.01, bf16=False):
    """optimizers::SGD::step (nt/nn/Optimizers.cpp:8-17) on one parameter: every whole-tensor operation of the
    reference rounds to the tensor's dtype, which numpy's typed arithmetic reproduces.  Returns the new parameter."""
    rnd, c = _typed_ops(param.dtype, bf16)
    g = rnd(_clamp10(grad, c) * c(lr))
    return rnd(param - g)


def adam_step(param, grad, m, v, lr=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, t=0, bf16=False):
    """optimizers::Adam::step (nt/nn/Optimizers.cpp:68-98), operation by operation as written there (the moment
    estimates are scaled by the gradient; the step counter t stays where the caller has it, 0 in the reference).
    Returns (param, m, v)."""
    rnd, c = _typed_ops(param.dtype, bf16)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        m1 = rnd(m * c(beta1))
        m1 = rnd(m1 + c(1 - beta1))
        m1 = rnd(m1 * grad)
        g2 = rnd(grad * grad)
        v1 = rnd(v * c(beta2))
        v1 = rnd(v1 + c(1 - beta2))
        v1 = rnd(v1 * g2)
        m_hat = rnd(m1 / c((1 - beta1) ** t))
        v_hat = rnd(v1 / c((1 - beta2) ** t))
        num = rnd(c(lr) * m_hat)
        den = rnd(rnd(np.sqrt(v_hat)) + c(epsilon))
        u = _clamp10(rnd(num / den), c)
        return rnd(param - u), m1, v1
