"""Grouped conv2d, conv1d, conv3d and the transposed convolutions against the reference's own golden vectors
(tests/src/conv_autograd_test.cpp:126-240 conv1d, :284-360 grouped conv2d, :376-500 conv3d, :556-960 conv_transpose1d/2d/3d; the
vectors were generated there with PyTorch and are compared with allclose).  CPU tests pin the oracle; GPU tests
run the same cases through the library."""
import os

import numpy as np
import pytest

from conftest import REF_GOLDEN

RTOL, ATOL = 1e-5, 1e-8   # nt::allclose defaults (nt/functional/tensor_files/compare.h:34), as the reference's tests use them


def g(name):
    return np.load(os.path.join(REF_GOLDEN, name + ".npy"))


def close(a, b):
    return a.shape == b.shape and np.allclose(a, b, rtol=RTOL, atol=ATOL)


CONV2D_GROUPED = [("_grouped", dict(stride=1, groups=2)), ("_grouped_batched", dict(stride=1, groups=2))]
CONV1D = [("", dict(stride=1, padding=1)), ("_batched", dict(stride=1, padding=1)),
          ("_grouped", dict(stride=1, groups=2)), ("_grouped_batched", dict(stride=1, groups=2))]
TRANSPOSE1D = [("", dict(stride=2, output_padding=1)), ("_batched", dict(stride=2, output_padding=1, padding=1)),
               ("_grouped", dict(stride=1, groups=2, padding=1)), ("_grouped_batched", dict(stride=1, groups=2, padding=1)),
               ("_grouped_bigger", dict(stride=1, groups=5, padding=1))]
CONV3D = [("", dict(stride=1, padding=1)), ("_grouped", dict(stride=1, groups=2)), ("_grouped_batched", dict(stride=1, groups=2))]
TRANSPOSE3D = [("", dict(stride=2, output_padding=1)), ("_grouped_batched", dict(stride=1, groups=2, padding=1))]
TRANSPOSE2D = [("", dict(stride=2, output_padding=1)), ("_batched", dict(stride=2, output_padding=1, padding=1)),
               ("_grouped", dict(stride=1, groups=5, padding=1)), ("_grouped_batched", dict(stride=1, groups=2, padding=1))]


def family(name, ext):
    return tuple(g("%s_%s%s" % (name, s, ext)) for s in ("input", "weight", "output", "grad", "xgrad", "wgrad"))


# ---------------------------------------------------------------------------------------------- oracle (CPU)
@pytest.mark.parametrize("ext,kw", CONV2D_GROUPED)
def test_oracle_grouped_conv2d(oracle, ext, kw):
    x, w, out, grad, xg, wg = family("conv2d", ext)
    assert close(oracle.conv2d(x, w, **kw), out)
    dx, dw = oracle.conv2d_backward(x, w, grad, **kw)
    assert close(dx, xg) and close(dw, wg)


@pytest.mark.parametrize("ext,kw", CONV1D)
def test_oracle_conv1d(oracle, ext, kw):
    x, w, out, grad, xg, wg = family("conv1d", ext)
    assert close(oracle.conv1d(x, w, **kw).reshape(out.shape), out)


@pytest.mark.parametrize("ext,kw", TRANSPOSE2D)
def test_oracle_conv_transpose2d(oracle, ext, kw):
    x, w, out, grad, xg, wg = family("conv_transpose2d", ext)
    assert close(oracle.conv_transpose2d(x, w, **kw), out)
    dx, dw = oracle.conv_transpose2d_backward(x, w, grad, **kw)
    assert close(dx, xg) and close(dw, wg)


@pytest.mark.parametrize("ext,kw", CONV3D)
def test_oracle_conv3d(oracle, ext, kw):
    x, w, out, grad, xg, wg = family("conv3d", ext)
    assert close(oracle.conv3d(x, w, **kw), out)
    dx, dw = oracle.conv3d_backward(x, w, grad, **kw)
    assert close(dx, xg) and close(dw, wg)


@pytest.mark.parametrize("ext,kw", TRANSPOSE3D)
def test_oracle_conv_transpose3d(oracle, ext, kw):
    x, w, out, grad, xg, wg = family("conv_transpose3d", ext)
    assert close(oracle.conv_transpose3d(x, w, **kw), out)
    dx, dw = oracle.conv_transpose3d_backward(x, w, grad, **kw)
    assert close(dx, xg) and close(dw, wg)


# ---------------------------------------------------------------------------------------------- library (GPU)
@pytest.fixture(scope="module")
def api():
    from neurotensor_b200 import api as a
    return a


@pytest.mark.gpu
@pytest.mark.parametrize("ext,kw", CONV2D_GROUPED)
def test_grouped_conv2d_golden(api, ext, kw):
    from gpu_util import dev, host
    x, w, out, grad, xg, wg = family("conv2d", ext)
    assert close(host(api.conv2d(dev(x), dev(w), **kw)), out)
    dx, dw = api.conv2d_backward(dev(x), dev(w), dev(grad), **kw)
    assert close(host(dx), xg) and close(host(dw), wg)


@pytest.mark.gpu
@pytest.mark.parametrize("ext,kw", CONV1D)
def test_conv1d_golden(api, ext, kw):
    from gpu_util import dev, host
    x, w, out, grad, xg, wg = family("conv1d", ext)
    assert close(host(api.conv1d(dev(x), dev(w), **kw)).reshape(out.shape), out)
    dx, dw = api.conv1d_backward(dev(x), dev(w), dev(grad), **kw)
    assert close(host(dx).reshape(xg.shape), xg) and close(host(dw).reshape(wg.shape), wg)


@pytest.mark.gpu
@pytest.mark.parametrize("ext,kw", TRANSPOSE1D)
def test_conv_transpose1d_golden(api, ext, kw):
    from gpu_util import dev, host
    x, w, out, grad, xg, wg = family("conv_transpose1d", ext)
    assert close(host(api.conv_transpose1d(dev(x), dev(w), **kw)).reshape(out.shape), out)
    dx, dw = api.conv_transpose1d_backward(dev(x), dev(w), dev(grad), **kw)
    assert close(host(dx).reshape(xg.shape), xg) and close(host(dw).reshape(wg.shape), wg)


@pytest.mark.gpu
@pytest.mark.parametrize("ext,kw", TRANSPOSE2D)
def test_conv_transpose2d_golden(api, ext, kw):
    from gpu_util import dev, host
    x, w, out, grad, xg, wg = family("conv_transpose2d", ext)
    assert close(host(api.conv_transpose2d(dev(x), dev(w), **kw)), out)
    dx, dw = api.conv_transpose2d_backward(dev(x), dev(w), dev(grad), **kw)
    assert close(host(dx), xg) and close(host(dw), wg)


@pytest.mark.gpu
@pytest.mark.parametrize("ext,kw", CONV3D)
def test_conv3d_golden(api, ext, kw):
    from gpu_util import dev, host
    x, w, out, grad, xg, wg = family("conv3d", ext)
    assert close(host(api.conv3d(dev(x), dev(w), **kw)), out)
    dx, dw = api.conv3d_backward(dev(x), dev(w), dev(grad), **kw)
    assert close(host(dx), xg) and close(host(dw), wg)


@pytest.mark.gpu
@pytest.mark.parametrize("ext,kw", TRANSPOSE3D)
def test_conv_transpose3d_golden(api, ext, kw):
    from gpu_util import dev, host
    x, w, out, grad, xg, wg = family("conv_transpose3d", ext)
    assert close(host(api.conv_transpose3d(dev(x), dev(w), **kw)), out)
    dx, dw = api.conv_transpose3d_backward(dev(x), dev(w), dev(grad), **kw)
    assert close(host(dx), xg) and close(host(dw), wg)


@pytest.mark.gpu
def test_unfold3d_bit_exact_and_conv3d_f16(api, oracle):
    """ntb200_im2col3d is a pure gather (bit-exact for any geometry); Float16 conv3d goes to the tensor cores."""
    import ctypes
    import torch
    from gpu_util import dev, host, normal
    from neurotensor_b200 import _lib
    rng = np.random.default_rng(37)
    x = normal(rng, (2, 5, 7, 9, 8), np.float32)
    k3, s3, p3, d3 = (2, 3, 2), (2, 1, 2), (1, 2, 0), (1, 2, 2)
    exp = oracle.unfold3d(x, k3, d3, p3, s3)
    geom = api._geom3(2, 5, (7, 9, 8), 1, 1, k3, s3, p3, d3)
    col = torch.empty(exp.shape, dtype=torch.float32, device="cuda")
    xd = dev(x)
    _lib.check(_lib.lib().ntb200_im2col3d(_lib.F32, xd.data_ptr(), col.data_ptr(), ctypes.byref(geom), None))
    assert np.array_equal(host(col), exp)
    back = torch.empty_like(xd)
    _lib.check(_lib.lib().ntb200_col2im3d(_lib.F32, col.data_ptr(), back.data_ptr(), ctypes.byref(geom), None))
    assert np.allclose(host(back), oracle.unfold3d_backward(exp, (7, 9, 8), k3, d3, p3, s3), rtol=1e-5, atol=1e-6)
    xh = normal(rng, (2, 16, 6, 8, 8), np.float16)
    wh = normal(rng, (24, 16, 3, 3, 3), np.float16, (1.0 / (16 * 27)) ** 0.5)
    got = host(api.conv3d(dev(xh), dev(wh), stride=1, padding=1))
    expc = oracle.conv3d(xh.astype(np.float32), wh.astype(np.float32), 1, 1, 1)
    assert oracle.rel_fro(got, expc) <= 2e-3


@pytest.mark.gpu
def test_grouped_and_transposed_f16_against_oracle(api, oracle):
    """Float16 on the tensor cores: grouped conv2d (column route per group) and a stride-1 transposed convolution
    (implicit convolution with the flipped kernel), against the oracle evaluated in Float32."""
    from gpu_util import dev, host, normal
    rng = np.random.default_rng(31)
    x = normal(rng, (3, 128, 12, 16), np.float16)
    w = normal(rng, (96, 32, 3, 3), np.float16, (1.0 / (32 * 9)) ** 0.5)
    got = host(api.conv2d(dev(x), dev(w), stride=1, padding=1, groups=4))
    exp = oracle.conv2d(x.astype(np.float32), w.astype(np.float32), 1, 1, 1, groups=4)
    assert oracle.rel_fro(got, exp) <= 2e-3
    xt = normal(rng, (2, 64, 10, 16), np.float16)
    wt = normal(rng, (64, 128, 3, 3), np.float16, (1.0 / (64 * 9)) ** 0.5)
    got_t = host(api.conv_transpose2d(dev(xt), dev(wt), stride=1, padding=1))
    exp_t = oracle.conv_transpose2d(xt.astype(np.float32), wt.astype(np.float32), stride=1, padding=1)
    assert got_t.shape == exp_t.shape and oracle.rel_fro(got_t, exp_t) <= 2e-3


@pytest.mark.gpu
def test_grouped_errors(api):
    import torch
    x = torch.zeros((1, 6, 8, 8), device="cuda")
    with pytest.raises(ValueError):
        api.conv2d(x, torch.zeros((4, 3, 3, 3), device="cuda"), groups=4)       # 6 channels do not split into 4 groups
    with pytest.raises(ValueError):
        api.conv2d(x, torch.zeros((4, 3, 3, 3), device="cuda"), groups=3)       # kernel channels * groups != channels
    with pytest.raises(ValueError):
        api.conv_transpose2d(x, torch.zeros((6, 2, 3, 3), device="cuda"), stride=1, output_padding=1)


# ---------------------------------------------------------------------------------------------- convnd
def _direct_convnd(x, w, dim, s, p, d, groups):
    """Definition of the N-D cross-correlation, summed in float64 tap by tap: the check of the column-matrix chain."""
    b, c = x.shape[:2]
    cout, cg = w.shape[:2]
    k = w.shape[2:]
    size = x.shape[2:]
    o = tuple((size[i] + 2 * p[i] - d[i] * (k[i] - 1) - 1) // s[i] + 1 for i in range(dim))
    xp = np.zeros((b, c) + tuple(size[i] + 2 * p[i] for i in range(dim)))
    xp[(slice(None), slice(None)) + tuple(slice(p[i], p[i] + size[i]) for i in range(dim))] = x
    out = np.zeros((b, cout) + o)
    coutg = cout // groups
    for gi in range(groups):
        for tap in np.ndindex(*k):
            src = tuple(slice(tap[i] * d[i], tap[i] * d[i] + (o[i] - 1) * s[i] + 1, s[i]) for i in range(dim))
            patch = xp[(slice(None), slice(gi * cg, (gi + 1) * cg)) + src]            # [b, cg, o...]
            wt = w[(slice(gi * coutg, (gi + 1) * coutg), slice(None)) + tap]          # [coutg, cg]
            out[:, gi * coutg:(gi + 1) * coutg] += np.einsum("bc...,oc->bo...", patch, wt.astype(np.float64))
    return out


CONVND_4D = [  # shapes of the reference's own ConvND (N = 4) cases, tests/src/conv_autograd_test.cpp:502-545, spatial extent reduced
    ((1, 3, 6, 6, 6, 6), (4, 3, 3, 3, 3, 3), dict(stride=1, padding=1, groups=1)),
    ((1, 4, 5, 5, 5, 5), (4, 2, 3, 3, 3, 3), dict(stride=1, padding=0, groups=2)),
    ((3, 4, 5, 5, 5, 5), (4, 2, 3, 3, 3, 3), dict(stride=1, padding=0, groups=2)),
    ((2, 2, 6, 5, 7, 6), (6, 1, 2, 3, 2, 3), dict(stride=(1, 2, 1, 2), padding=(1, 0, 2, 1), dilation=(2, 1, 1, 2), groups=2)),
]


def test_oracle_convnd_equals_the_fixed_rank_oracles(oracle):
    """unfoldnd in 1, 2 and 3 dimensions is unfold1d / 2d / 3d (the reference's own assertion,
    tests/src/col_im_tests.cpp:47-83), so convnd there must equal the golden-pinned conv1d / conv2d / conv3d."""
    rng = np.random.default_rng(3)
    x3 = rng.standard_normal((2, 4, 7, 6, 5)).astype(np.float32)
    w3 = rng.standard_normal((6, 2, 3, 2, 3)).astype(np.float32)
    kw = dict(stride=(1, 2, 1), padding=(1, 0, 2), dilation=(1, 1, 2), groups=2)
    assert np.array_equal(oracle.convnd(x3, w3, 3, **kw), oracle.conv3d(x3, w3, **kw))
    g3 = rng.standard_normal(oracle.conv3d(x3, w3, **kw).shape).astype(np.float32)
    for a, b in zip(oracle.convnd_backward(x3, w3, g3, 3, **kw), oracle.conv3d_backward(x3, w3, g3, **kw)):
        assert np.array_equal(a, b)
    x2 = rng.standard_normal((2, 3, 9, 8)).astype(np.float32)
    w2 = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    assert np.array_equal(oracle.convnd(x2, w2, 2, 2, 1, 1), oracle.conv2d(x2, w2, 2, 1, 1))
    x1 = rng.standard_normal((2, 4, 19)).astype(np.float32)
    w1 = rng.standard_normal((6, 2, 3)).astype(np.float32)
    assert np.array_equal(oracle.convnd(x1, w1, 1, 2, 1, 1, groups=2).reshape(2, 6, -1), oracle.conv1d(x1, w1, 2, 1, 1, groups=2).reshape(2, 6, -1))
    xt = rng.standard_normal((2, 4, 3, 4, 3)).astype(np.float32)
    wt = rng.standard_normal((4, 3, 2, 3, 2)).astype(np.float32)
    kt = dict(stride=(2, 1, 2), padding=(0, 1, 0), output_padding=(1, 0, 1), dilation=1, groups=2)
    assert np.array_equal(oracle.conv_transposend(xt, wt, 3, **kt), oracle.conv_transpose3d(xt, wt, **kt))


@pytest.mark.parametrize("xs,ws,kw", CONVND_4D)
def test_oracle_convnd_4d_against_the_definition(oracle, xs, ws, kw):
    rng = np.random.default_rng(5)
    x = rng.uniform(0, 3, xs).astype(np.float32)
    w = rng.uniform(0, 3, ws).astype(np.float32)
    t = lambda v: tuple(v) if isinstance(v, tuple) else (v,) * 4
    exp = _direct_convnd(x, w, 4, t(kw["stride"]), t(kw["padding"]), t(kw.get("dilation", 1)), kw["groups"])
    got = oracle.convnd(x, w, 4, **kw)
    assert got.shape == exp.shape and np.allclose(got, exp, rtol=1e-5, atol=1e-5)
    # the adjoint identities <conv(x), g> = <x, d_image> = <w, d_kernel> hold for the backward chain
    grad = rng.uniform(0, 1, got.shape).astype(np.float32)
    dx, dw = oracle.convnd_backward(x, w, grad, 4, **kw)
    lhs = float(np.sum(got.astype(np.float64) * grad))
    assert abs(float(np.sum(x.astype(np.float64) * dx)) - lhs) <= 1e-4 * abs(lhs)
    assert abs(float(np.sum(w.astype(np.float64) * dw)) - lhs) <= 1e-4 * abs(lhs)


@pytest.mark.gpu
@pytest.mark.parametrize("xs,ws,kw", CONVND_4D + [((1, 3, 16, 16, 16, 16), (4, 3, 3, 3, 3, 3), dict(stride=1, padding=1, groups=1))])
def test_convnd_4d(api, oracle, xs, ws, kw):
    """convnd with N = 4 (the reference's ConvND cases, the first at its full 16^4 extent) against the oracle at the
    reference's allclose tolerance, forward and both gradients."""
    from gpu_util import dev, host
    rng = np.random.default_rng(7)
    x = rng.uniform(0, 3, xs).astype(np.float32)
    w = rng.uniform(0, 3, ws).astype(np.float32)
    exp = oracle.convnd(x, w, 4, **kw)
    got = host(api.convnd(dev(x), dev(w), 4, **kw))
    assert close(got, exp)
    grad = rng.uniform(0, 1, exp.shape).astype(np.float32)
    edx, edw = oracle.convnd_backward(x, w, grad, 4, **kw)
    dx, dw = api.convnd_backward(dev(x), dev(w), dev(grad), 4, **kw)
    assert close(host(dx), edx)
    # the kernel gradient is a sum over all output positions of all-positive products (uniform inputs, as in the
    # reference's case): two Float32 chains of that length in different orders differ by about sqrt(L) roundings, which
    # passes the reference's 1e-5 up to L = 4096 and needs 4 sqrt(L) 2^-24 at the full 16^4 extent (L = 65536: 6e-5)
    length = int(np.prod(exp.shape[2:]))
    assert np.allclose(host(dw), edw, rtol=max(RTOL, 4.0 * length ** 0.5 * 2.0 ** -24), atol=1e-8)


@pytest.mark.gpu
def test_convnd_equals_fixed_rank_calls_and_unfoldnd_is_a_gather(api, oracle):
    """N = 1, 2, 3 give what conv1d / conv2d / conv3d give (tests/src/col_im_tests.cpp:47-117 assert this of unfoldnd),
    unfoldnd is bit-exact for any geometry, integer images included, and conv_transposend equals conv_transpose3d."""
    import torch
    from gpu_util import dev, host, normal
    rng = np.random.default_rng(11)
    x3 = normal(rng, (2, 4, 7, 6, 5), np.float32)
    w3 = normal(rng, (6, 2, 3, 2, 3), np.float32)
    kw = dict(stride=(1, 2, 1), padding=(1, 0, 2), dilation=(1, 1, 2), groups=2)
    a, b = host(api.convnd(dev(x3), dev(w3), 3, **kw)), host(api.conv3d(dev(x3), dev(w3), **kw))
    near = lambda u, v: u.shape == v.shape and np.allclose(u, v, rtol=1e-5, atol=1e-6)
    assert np.array_equal(a, b) and near(a, oracle.conv3d(x3, w3, **kw))
    x2 = normal(rng, (2, 3, 9, 8), np.float32)
    w2 = normal(rng, (4, 3, 3, 3), np.float32)
    assert near(host(api.convnd(dev(x2), dev(w2), 2, 2, 1, 1)), oracle.conv2d(x2, w2, 2, 1, 1))
    x1 = normal(rng, (2, 4, 19), np.float32)
    w1 = normal(rng, (6, 2, 3), np.float32)
    assert near(host(api.convnd(dev(x1), dev(w1), 1, 2, 1, 1, groups=2)), oracle.conv1d(x1, w1, 2, 1, 1, groups=2).reshape(2, 6, -1))
    # unfoldnd: a pure gather, any element size
    x4 = rng.integers(-100, 100, (1, 2, 6, 6, 6, 6)).astype(np.int32)
    k4, d4, p4, s4 = (3, 3, 3, 3), 1, (1, 1, 1, 1), (1, 1, 2, 2)   # tests/src/col_im_autograd_test.cpp:183-190
    exp = oracle.unfoldnd(x4, 4, k4, d4, p4, s4)
    assert np.array_equal(host(api.unfoldnd(dev(x4), 4, k4, d4, p4, s4)), exp)
    xf = x4.astype(np.float32)
    col = api.unfoldnd(dev(xf), 4, k4, d4, p4, s4)
    back = host(api.unfoldnd_backward(col, 4, (6, 6, 6, 6), k4, d4, p4, s4))
    assert np.array_equal(back, oracle.unfoldnd_backward(exp.astype(np.float32), 4, (6, 6, 6, 6), k4, d4, p4, s4))   # small integers: exact
    xt = normal(rng, (2, 4, 3, 4, 3), np.float32)
    wt = normal(rng, (4, 3, 2, 3, 2), np.float32)
    kt = dict(stride=(2, 1, 2), padding=(0, 1, 0), output_padding=(1, 0, 1), dilation=1, groups=2)
    got = host(api.conv_transposend(dev(xt), dev(wt), 3, **kt))
    assert np.array_equal(got, host(api.conv_transpose3d(dev(xt), dev(wt), **kt)))   # same taps in the same order
    # normal inputs cancel: sums near zero differ from the oracle's order by an absolute, not a relative, amount
    assert np.allclose(got, oracle.conv_transpose3d(xt, wt, **kt), rtol=1e-5, atol=1e-6)
    gt = normal(rng, got.shape, np.float32)
    edx, edw = oracle.conv_transpose3d_backward(xt, wt, gt, **kt)
    dx, dw = api.conv_transposend_backward(dev(xt), dev(wt), dev(gt), 3, **kt)
    assert np.allclose(host(dx), edx, rtol=1e-5, atol=1e-6) and np.allclose(host(dw), edw, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        api.convnd(dev(x3), dev(w3), 0)
    with pytest.raises(ValueError):
        api.convnd(dev(x3), dev(w3), 3, stride=0)
    xh = normal(rng, (2, 16, 4, 5, 4, 5), np.float16)
    wh = normal(rng, (24, 16, 3, 3, 3, 3), np.float16, (1.0 / (16 * 81)) ** 0.5)
    goth = host(api.convnd(dev(xh), dev(wh), 4, stride=1, padding=1))
    assert oracle.rel_fro(goth, oracle.convnd(xh.astype(np.float32), wh.astype(np.float32), 4, 1, 1, 1)) <= 2e-3
