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


def _pool_state(L):
    """(bytes handed out by the device's stream-ordered pool, their high-water mark since the reset just made,
    scratch blocks the library has handed to its own kernels so far)"""
    lib = L.lib()
    used, high, acq = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
    L.check(lib.ntb200_device_pool_usage(ctypes.byref(used), ctypes.byref(high), None, 1))
    L.check(lib.ntb200_scratch_stats(None, ctypes.byref(acq), None))
    return used.value, high.value, acq.value


def _static_only(L, code, x, w, geom):
    lib = L.lib()
    bsz, ch, h, wd = x.shape
    cout, _, kh, kw = w.shape
    sh, sw, ph, pw, dh, dw = geom
    ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (wd + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    need = lib.ntb200_conv2d_workspace_bytes(code, bsz, ch, h, wd, kh, kw, sh, sw, ph, pw, dh, dw)
    assert 0 < need <= L.CONV2D_STATIC_SCRATCH_BYTES
    got = torch.zeros((bsz, cout, ho, wo), dtype=x.dtype, device="cuda")
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    used0, _, acq0 = _pool_state(L)
    L.check(lib.ntb200_conv2d_static_scratch(code, x.data_ptr(), w.data_ptr(), got.data_ptr(), bsz, ch, h, wd, cout,
                                             kh, kw, sh, sw, ph, pw, dh, dw, s))
    route = L.last_route()
    torch.cuda.synchronize()
    used1, high1, acq1 = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
    L.check(lib.ntb200_device_pool_usage(ctypes.byref(used1), ctypes.byref(high1), None, 0))
    L.check(lib.ntb200_scratch_stats(None, ctypes.byref(acq1), None))
    # nothing was taken from the pool during the call, not even for a moment, and no scratch block was handed out
    assert used1.value == used0, (used0, used1.value)
    assert high1.value <= used0, (used0, high1.value)
    assert acq1.value == acq0, "the call took a scratch block (%d -> %d)" % (acq0, acq1.value)
    return got, route


NON_ALLOCATING_ROUTES = {"simt", "umma_f16", "umma_bf16", "umma_i8", "conv2d-implicit-umma-pair"}


def test_static_scratch_allocates_nothing_on_the_routes_that_would():
    """Problems that fit the built-in array but whose GEMM, through ntb200_conv2d, takes a route with scratch of its
    own (Float32 as three TF32 products, Int32 limb planes, Float16 K slices).  Through this entry point they must
    allocate nothing, and still give the reference's result."""
    from neurotensor_b200 import _lib as L
    from oracle import oracle
    rng = np.random.default_rng(77)
    # Float32, 1.16e8 multiply-adds (the automatic route would split the operands into hi/lo copies)
    x = torch.from_numpy(rng.standard_normal((1, 64, 56, 56)).astype(np.float32)).cuda()
    w = torch.from_numpy((rng.standard_normal((64, 64, 3, 3)) / 24).astype(np.float32)).cuda()
    got, route = _static_only(L, L.F32, x, w, (1, 1, 1, 1, 1, 1))
    assert route in NON_ALLOCATING_ROUTES, route
    assert np.array_equal(got.cpu().numpy(), oracle.conv2d(x.cpu().numpy(), w.cpu().numpy(), stride=1, padding=1))   # one chain per output: bit-exact
    # Float32, batched: 8 x 64 x 28 x 28 against 128 filters (a 14 MB column matrix)
    x = torch.from_numpy(rng.standard_normal((8, 64, 28, 28)).astype(np.float32)).cuda()
    w = torch.from_numpy((rng.standard_normal((128, 64, 3, 3)) / 24).astype(np.float32)).cuda()
    got, route = _static_only(L, L.F32, x, w, (1, 1, 1, 1, 1, 1))
    assert route in NON_ALLOCATING_ROUTES, route
    assert np.array_equal(got.cpu().numpy(), oracle.conv2d(x.cpu().numpy(), w.cpu().numpy(), stride=1, padding=1))
    # Int32 above 6e7 multiply-adds (the automatic route would write limb planes)
    xi = torch.from_numpy(rng.integers(-1000, 1000, (4, 32, 32, 32)).astype(np.int32)).cuda()
    wi = torch.from_numpy(rng.integers(-1000, 1000, (64, 32, 3, 3)).astype(np.int32)).cuda()
    got, route = _static_only(L, L.I32, xi, wi, (1, 1, 1, 1, 1, 1))
    assert route in NON_ALLOCATING_ROUTES, route
    assert np.array_equal(got.cpu().numpy(), oracle.conv2d(xi.cpu().numpy(), wi.cpu().numpy(), stride=1, padding=1))
    # Float16, one image, stride 2 (no implicit route), K = 512 * 9 = 4608: the automatic route would cut K into slices.
    # At this depth fp32 accumulation is 2.5e-3 from the reference's fp16 rounding every 16 k by construction (beyond
    # K of about 2300 the two drift past 2e-3), so the bar is on the value accumulated in fp32 and rounded once; the
    # distance to the reference-faithful oracle is measured and must be the expected one.
    xh = torch.from_numpy((rng.standard_normal((1, 512, 28, 28))).astype(np.float16)).cuda()
    wh = torch.from_numpy((rng.standard_normal((256, 512, 3, 3)) / 68).astype(np.float16)).cuda()
    got, route = _static_only(L, L.F16, xh, wh, (2, 2, 1, 1, 1, 1))
    assert route in NON_ALLOCATING_ROUTES, route
    wide = torch.nn.functional.conv2d(xh.double(), wh.double(), stride=2, padding=1).float().half()
    d_wide = oracle.rel_fro(got.cpu().numpy(), wide.cpu().numpy())
    d_ref = oracle.rel_fro(got.cpu().numpy(), oracle.conv2d(xh.cpu().numpy(), wh.cpu().numpy(), stride=2, padding=1))
    assert d_wide <= 2e-3 and d_ref <= 3.2e-3, (d_wide, d_ref)
    # Float16 with two filters (the automatic route would stream the weights and leave partial sums in scratch)
    wt = torch.from_numpy((rng.standard_normal((2, 512, 3, 3)) / 68).astype(np.float16)).cuda()
    got, route = _static_only(L, L.F16, xh, wt, (2, 2, 1, 1, 1, 1))
    assert route in NON_ALLOCATING_ROUTES, route
    wide = torch.nn.functional.conv2d(xh.double(), wt.double(), stride=2, padding=1).float().half()
    assert oracle.rel_fro(got.cpu().numpy(), wide.cpu().numpy()) <= 2e-3


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
