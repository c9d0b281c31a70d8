"""ntb200_conv2d_static_scratch: the conv2d variant for users who cannot allocate device memory (their
application owns the whole device heap, or forbids itself cudaMalloc because it synchronises the device).
It must give exactly what ntb200_conv2d gives with a caller-provided workspace, on repeated calls that share
the library's built-in scratch array, and must refuse problems whose column matrix does not fit.

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
The test makes no assumption about earlier tests: it runs the same alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(L, code, x, w, geom):
    """(result of the workspace entry point, result of the built-in-scratch entry point)"""
    lib = L.lib()
    bsz, ch, h, wd = x.shape
    cout, _, kh, kw = w.shape
    sh, sw, ph, pw, dh, dw = geom
    ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (wd + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.ntb200_conv2d_workspace_bytes(code, bsz, ch, h, wd, kh, kw, sh, sw, ph, pw, dh, dw)
    assert 0 < need <= L.CONV2D_STATIC_SCRATCH_BYTES
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    ref = torch.full((bsz, cout, ho, wo), float("nan"), dtype=x.dtype, device="cuda")
    got = torch.full_like(ref, float("nan"))
    L.check(lib.ntb200_conv2d(code, x.data_ptr(), w.data_ptr(), ref.data_ptr(), ws.data_ptr(), bsz, ch, h, wd, cout,
                              kh, kw, sh, sw, ph, pw, dh, dw, s))
    L.check(lib.ntb200_conv2d_static_scratch(code, x.data_ptr(), w.data_ptr(), got.data_ptr(), bsz, ch, h, wd, cout,
                                             kh, kw, sh, sw, ph, pw, dh, dw, s))
    torch.cuda.synchronize()
    return ref, got


def test_static_scratch_conv2d_matches_workspace_conv2d_twice():
    from neurotensor_b200 import _lib as L
    gen = torch.Generator(device="cuda").manual_seed(123)
    # call 1: Float16 on the tensor cores, padded 3x3; the scratch receives the channels-last copy of the input and
    # the reordered weights
    x1 = torch.randn((4, 64, 28, 28), generator=gen, device="cuda").half()
    w1 = (torch.randn((96, 64, 3, 3), generator=gen, device="cuda") / 24).half()
    ref1, got1 = _both(L, L.F16, x1, w1, (1, 1, 1, 1, 1, 1))
    assert L.last_route() == "conv2d-implicit-umma-pair"
    assert not torch.isnan(got1).any()
    assert torch.equal(got1, ref1)          # same kernels on the same data: identical bits
    # call 2 straight after, a smaller Float32 problem with different geometry: the scratch still holds call 1's
    # data, none of which may show up in the result
    x2 = torch.randn((2, 5, 17, 13), generator=gen, device="cuda")
    w2 = torch.randn((7, 5, 2, 4), generator=gen, device="cuda")
    ref2, got2 = _both(L, L.F32, x2, w2, (2, 1, 0, 3, 1, 2))
    assert not torch.isnan(got2).any()
    assert torch.equal(got2, ref2)
    # and call 1 again gives call 1's answer again
    ref3, got3 = _both(L, L.F16, x1, w1, (1, 1, 1, 1, 1, 1))
    assert torch.equal(got3, ref1)
    # against the CPU oracle too, within the Float16 bar the other tests use
    from oracle import oracle
    exp = oracle.conv2d(x1.cpu().numpy(), w1.cpu().numpy(), stride=1, padding=1)
    assert oracle.rel_fro(got1.cpu().numpy(), exp) <= 2e-3
    exp2 = oracle.conv2d(x2.cpu().numpy(), w2.cpu().numpy(), stride=(2, 1), padding=(0, 3), dilation=(1, 2))
    assert np.array_equal(got2.cpu().numpy(), exp2)


def test_static_scratch_refuses_what_does_not_fit():
    from neurotensor_b200 import _lib as L
    lib = L.lib()
    x = torch.zeros((32, 256, 56, 56), dtype=torch.float16, device="cuda")   # column matrix: 462 MB
    w = torch.zeros((256, 256, 3, 3), dtype=torch.float16, device="cuda")
    out = torch.zeros((32, 256, 56, 56), dtype=torch.float16, device="cuda")
    before = L.launch_count()
    rc = lib.ntb200_conv2d_static_scratch(L.F16, x.data_ptr(), w.data_ptr(), out.data_ptr(), 32, 256, 56, 56, 256, 3, 3,
                                          1, 1, 1, 1, 1, 1, None)
    assert rc == L.ERR_INVALID_ARG
    msg = lib.ntb200_last_error_string().decode()
    assert "462422016" in msg and str(L.CONV2D_STATIC_SCRATCH_BYTES) in msg
    assert L.launch_count() == before      # nothing was launched
