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
