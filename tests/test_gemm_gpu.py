"""GPU parity of matmult against the CPU oracle, through the C ABI (ctypes -> libntb200.so).

Bars: integers bit-exact; Float32 bit-exact on the CUDA-core route (one ascending-k FMA chain, like the
reference) and in any case within 1e-5 relative Frobenius error; Float16 / BFloat16 within 2e-3 relative
Frobenius error of the reference-faithful oracle (fp32 accumulate on tensor cores), and bit-exact on the
CUDA-core route with per-K-tile rounding."""
import numpy as np
import pytest
import torch

from gpu_util import Codec, check_16bit, dev, host, integers, normal

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F16_TOL = 2e-3


@pytest.fixture(scope="module")
def api():
    from neurotensor_b200 import api as a
    return a


@pytest.fixture(scope="module")
def L():
    from neurotensor_b200 import _lib
    return _lib


FLAGS = [(False, False), (True, False), (False, True), (True, True)]


def operands(rng, m, k, n, ta, tb, dtype, scale=1.0, ints=None):
    sa = (k, m) if ta else (m, k)
    sb = (n, k) if tb else (k, n)
    if ints:
        return integers(rng, sa, dtype, *ints), integers(rng, sb, dtype, *ints)
    return normal(rng, sa, dtype, scale), normal(rng, sb, dtype, scale)


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (7, 5, 3), (64, 64, 64), (130, 47, 129), (257, 130, 255), (512, 300, 384)])
def test_f32_bit_exact(api, oracle, ta, tb, m, k, n):
    rng = np.random.default_rng(m * 1000 + k)
    a, b = operands(rng, m, k, n, ta, tb, np.float32)
    got = host(api.matmult(dev(a), dev(b), ta, tb))
    exp = oracle.matmult(a, b, ta, tb)
    assert np.array_equal(got, exp)


def test_f32_config_1024(api, oracle, L):
    """BASELINE config 0: Float32 1024^3, contiguous row-major, N(0,1).  The default route is the tensor-core
    kernel with three TF32 products per multiply (within the 1e-5 bar); the CUDA-core route is bit-exact."""
    rng = np.random.default_rng(1)
    a, b = normal(rng, (1024, 1024), np.float32), normal(rng, (1024, 1024), np.float32)
    exp = oracle.matmult(a, b)
    got = host(api.matmult(dev(a), dev(b)))
    assert L.last_route() == "umma_3xtf32"
    err = oracle.rel_fro(got, exp)
    assert err <= F32_TOL, err
    exact = host(api.matmult(dev(a), dev(b), route=L.ROUTE_SIMT))
    assert L.last_route() == "simt"
    assert np.array_equal(exact, exp)


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n", [(128, 32, 64), (257, 130, 255), (384, 1023, 640), (2048, 512, 2304)])
def test_f32_three_tf32_route(api, oracle, L, ta, tb, m, k, n):
    """Float32 on tensor cores: any strides (the split pass copies), K not a multiple of 4, M/N tails, pair tiles."""
    rng = np.random.default_rng(53 + m + k)
    a, b = operands(rng, m, k, n, ta, tb, np.float32)
    got = host(api.matmult(dev(a), dev(b), ta, tb, route=L.ROUTE_TENSOR))
    assert L.last_route() == "umma_3xtf32"
    err = oracle.rel_fro(got, oracle.matmult(a, b, ta, tb))
    assert err <= F32_TOL, err


def test_f32_three_tf32_bias_accumulate_and_shared_operand(api, oracle, L):
    rng = np.random.default_rng(59)
    x, w = normal(rng, (3, 200, 96), np.float32), normal(rng, (96, 136), np.float32)
    bias, c0 = normal(rng, (136,), np.float32), normal(rng, (3, 200, 136), np.float32)
    got = host(api.linear(dev(x), dev(w), dev(bias), route=L.ROUTE_TENSOR))
    assert L.last_route() == "umma_3xtf32"
    assert oracle.rel_fro(got, oracle.linear(x, w, bias)) <= F32_TOL
    out = dev(c0)
    api.matmult(dev(x), dev(w), out=out, route=L.ROUTE_TENSOR)
    assert oracle.rel_fro(host(out), c0 + oracle.matmult(x, w)) <= F32_TOL
    # values spanning many binades and exact zero rows keep their accuracy
    big = (normal(rng, (130, 64), np.float32) * np.exp2(rng.integers(-20, 20, (130, 64)))).astype(np.float32)
    big[1, :] = 0
    small = normal(rng, (64, 70), np.float32)
    got = host(api.matmult(dev(big), dev(small), route=L.ROUTE_TENSOR))
    exp = oracle.matmult(big, small)
    assert np.all(got[1] == 0) and np.isfinite(got).all()
    assert oracle.rel_fro(got, exp) <= F32_TOL
    # an infinite input stays non-finite (inf or NaN: inf x (hi + lo) may meet inf - inf); the CUDA-core route is exact
    big[0, 0] = np.inf
    got = host(api.matmult(dev(big), dev(small), route=L.ROUTE_TENSOR))
    assert not np.isfinite(got[0]).any() and np.isfinite(got[1:]).all()
    assert np.array_equal(host(api.matmult(dev(big), dev(small), route=L.ROUTE_SIMT)), oracle.matmult(big, small), equal_nan=True)


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n", [(128, 64, 256), (128, 128, 64), (256, 192, 512), (136, 200, 72), (384, 1024, 640)])
def test_f16_tensor_core_route(api, oracle, L, ta, tb, m, k, n):
    rng = np.random.default_rng(7 + m + k + n)
    a, b = operands(rng, m, k, n, ta, tb, np.float16, 0.5)
    got = host(api.matmult(dev(a), dev(b), ta, tb, route=L.ROUTE_TENSOR))
    assert L.last_route().startswith("umma_f16")      # one-pass kernel, or K slices inside a cluster for deep, small problems
    exp = oracle.matmult(a, b, ta, tb)
    wide = (a.T if ta else a).astype(np.float32) @ (b.T if tb else b).astype(np.float32)
    assert oracle.rel_fro(got, wide) <= 5e-4, "vs fp32-accumulate"
    assert oracle.rel_fro(got, exp) <= F16_TOL, "vs the reference-faithful oracle"


@pytest.mark.parametrize("ta,tb", FLAGS)
def test_f16_per_ktile_rounding_is_bit_exact(api, oracle, L, ta, tb):
    rng = np.random.default_rng(11)
    a, b = operands(rng, 70, 150, 90, ta, tb, np.float16, 0.5)
    got = host(api.matmult(dev(a), dev(b), ta, tb, f16_rounding=L.F16_ROUND_PER_KTILE))
    assert L.last_route() == "simt"
    exp = oracle.matmult(a, b, ta, tb)
    assert np.array_equal(got.view(np.uint16), exp.view(np.uint16))


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n", [(128, 64, 128), (200, 328, 136), (256, 512, 256)])
def test_bf16_tensor_core_route(api, oracle, L, ta, tb, m, k, n):
    rng = np.random.default_rng(13 + m)
    a32, b32 = operands(rng, m, k, n, ta, tb, np.float32)
    a, b = oracle.bf16_round(a32), oracle.bf16_round(b32)
    got = host(api.matmult(dev(a, True), dev(b, True), ta, tb, route=L.ROUTE_TENSOR))
    assert L.last_route().startswith("umma_bf16")
    exp = oracle.matmult(a, b, ta, tb, bf16=True)
    assert oracle.rel_fro(oracle.bf16_widen(got), oracle.bf16_widen(exp)) <= F16_TOL


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (144, 400, 272), (256, 1024, 512)])
@pytest.mark.parametrize("dt", [np.int8, np.uint8])
def test_int8_tensor_core_route_bit_exact(api, oracle, L, ta, tb, m, k, n, dt):
    rng = np.random.default_rng(17 + k)
    info = np.iinfo(dt)
    a, b = operands(rng, m, k, n, ta, tb, dt, ints=(info.min, info.max))
    got = host(api.matmult(dev(a), dev(b), ta, tb, route=L.ROUTE_TENSOR))
    assert L.last_route() == "umma_i8"
    assert np.array_equal(got, oracle.matmult(a, b, ta, tb))


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("dt", [np.int8, np.int16, np.int32, np.int64, np.uint8])
def test_integers_cuda_core_route_bit_exact(api, oracle, L, ta, tb, dt):
    rng = np.random.default_rng(19)
    info = np.iinfo(dt)
    a, b = operands(rng, 131, 77, 65, ta, tb, dt, ints=(info.min, info.max))
    got = host(api.matmult(dev(a), dev(b), ta, tb, route=L.ROUTE_SIMT))
    assert np.array_equal(got, oracle.matmult(a, b, ta, tb))


def test_f64(api, oracle):
    rng = np.random.default_rng(23)
    a, b = normal(rng, (90, 70), np.float64), normal(rng, (70, 50), np.float64)
    assert np.array_equal(host(api.matmult(dev(a), dev(b))), oracle.matmult(a, b))


def test_unaligned_fp16_falls_to_cuda_cores_not_cpu(api, oracle, L):
    """Row stride 2*67 bytes is not 16-byte aligned: TMA cannot stage it, the CUDA-core kernel runs."""
    rng = np.random.default_rng(29)
    a, b = normal(rng, (40, 67), np.float16, 0.5), normal(rng, (67, 33), np.float16, 0.5)
    got = host(api.matmult(dev(a), dev(b)))
    assert L.last_route() == "simt"
    assert oracle.rel_fro(got, oracle.matmult(a, b)) <= F16_TOL
    with pytest.raises(L.Ntb200Error):
        api.matmult(dev(a), dev(b), route=L.ROUTE_TENSOR)


def test_complex32_matmult(api, oracle, L):
    """Complex32 (pairs of Float16): lane-wise like Complex64, the running sums rounded to Float16 at the edges of the
    reference's K tile for this type, every 8 k-steps.  Bit for bit against the oracle (which is pinned on the compiled
    reference kernel for this type): 2-D, batched against a 2-D operand, both transposed views, C +=."""
    rng = np.random.default_rng(109)
    pairs = lambda shape: normal(rng, shape + (2,), np.float16, 0.5)
    as_c32 = lambda arr: torch.view_as_complex(torch.from_numpy(arr).cuda())
    back = lambda t: torch.view_as_real(t).cpu().numpy()
    a, b = pairs((3, 70, 45)), pairs((45, 133))
    got = api.matmult(as_c32(a), as_c32(b))
    assert L.last_route() == "simt" and got.dtype == torch.complex32
    assert np.array_equal(back(got), oracle.matmult_complex32(a, b))
    bt, at = pairs((133, 45)), pairs((3, 45, 70))
    assert np.array_equal(back(api.matmult(as_c32(a), as_c32(bt), transpose_b=True)), oracle.matmult_complex32(a, bt, transpose_b=True))
    assert np.array_equal(back(api.matmult(as_c32(at), as_c32(b), transpose_a=True)), oracle.matmult_complex32(at, b, transpose_a=True))
    # fp32 lanes rounded once would differ: the tile-edge rounding is really there
    once = np.stack([(a[0, ..., i].astype(np.float32) @ b[..., i].astype(np.float32)).astype(np.float16) for i in (0, 1)], axis=-1)
    assert not np.array_equal(back(got)[0], once)
    c0 = pairs((70, 133))
    out = as_c32(c0.copy())
    api.matmult(as_c32(a[0]), as_c32(b), out=out)
    exp = np.stack([oracle.matmult_into(np.ascontiguousarray(a[0, ..., i]), np.ascontiguousarray(b[..., i]), np.ascontiguousarray(c0[..., i]),
                                        bf16="c32-lane") for i in (0, 1)], axis=-1)
    assert np.array_equal(back(out), exp)


def test_transposed_view_is_not_copied(api, oracle, L):
    """b.transpose(-1,-2) is a stride swap (the reference flips the flag, matmult_cpu.cpp:268-273)."""
    rng = np.random.default_rng(31)
    a, bs = normal(rng, (4, 128, 192), np.float16, 0.3), normal(rng, (4, 256, 192), np.float16, 0.3)
    bview = dev(bs).transpose(-1, -2)
    assert not bview.is_contiguous()
    got = host(api.matmult(dev(a), bview, route=L.ROUTE_TENSOR))
    exp = oracle.matmult(a, bs, False, True)
    assert oracle.rel_fro(got, exp) <= F16_TOL
    # the same through flags
    got2 = host(api.matmult(dev(a), dev(bs), False, True, route=L.ROUTE_TENSOR))
    assert np.array_equal(got, got2)


def test_batched_and_repeated_operand(api, oracle):
    rng = np.random.default_rng(37)
    a = normal(rng, (3, 2, 33, 20), np.float32)
    b = normal(rng, (3, 2, 20, 17), np.float32)
    assert np.array_equal(host(api.matmult(dev(a), dev(b))), oracle.matmult(a, b))
    w = normal(rng, (20, 9), np.float32)     # 2-D operand repeated over the batch
    assert np.array_equal(host(api.matmult(dev(a), dev(w))), oracle.matmult(a, w))
    x = normal(rng, (33, 20), np.float32)
    assert np.array_equal(host(api.matmult(dev(x), dev(b))), oracle.matmult(x, b))


@pytest.mark.parametrize("dt,route", [(np.float32, "auto"), (np.int32, "auto"), (np.float16, "tensor"), (np.int8, "tensor")])
def test_out_variant_accumulates(api, oracle, L, dt, route):
    """matmult(a, b, out): out += a.b, the raw-pointer contract of nt_matmult."""
    rng = np.random.default_rng(41)
    if np.issubdtype(dt, np.integer):
        a, b, c = (integers(rng, s, dt, -9, 9) for s in ((128, 96), (96, 160), (128, 160)))
    else:
        a, b, c = (normal(rng, s, dt, 0.5) for s in ((128, 96), (96, 160), (128, 160)))
    out = dev(c)
    r = api.matmult(dev(a), dev(b), out=out, route=L.ROUTE_TENSOR if route == "tensor" else L.ROUTE_AUTO)
    assert r.data_ptr() == out.data_ptr()
    exp = c.copy()
    oracle.matmult_into(a, b, exp)
    if dt == np.float16:
        assert oracle.rel_fro(host(out), exp) <= F16_TOL
    else:
        assert np.array_equal(host(out), exp)


def test_raw_contract_and_pointer_tables(api, oracle, L):
    """ntb200_matmult / ntb200_matmult_batch with the reference's raw-pointer signature."""
    import ctypes
    rng = np.random.default_rng(43)
    a, b = normal(rng, (5, 40, 24), np.float32), normal(rng, (5, 24, 56), np.float32)
    da, db = dev(a), dev(b)
    dc = torch.zeros((5, 40, 56), dtype=torch.float32, device="cuda")
    lib = L.lib()
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    L.check(lib.ntb200_matmult(L.F32, da[0].data_ptr(), db[0].data_ptr(), dc[0].data_ptr(), 40, 24, 24, 56, 0, 0, s))
    exp = oracle.matmult(a, b)
    assert np.array_equal(host(dc[0]), exp[0])
    # equally spaced pointers -> one strided launch
    dc.zero_()
    arr = lambda t, order: (ctypes.c_void_p * 5)(*[t[i].data_ptr() for i in order])
    order = list(range(5))
    L.check(lib.ntb200_matmult_batch(L.F32, arr(da, order), arr(db, order), arr(dc, order), 5, 40, 24, 24, 56, 0, 0, s))
    assert np.array_equal(host(dc), exp)
    # shuffled pointers -> device pointer tables
    dc.zero_()
    order = [3, 0, 4, 1, 2]
    L.check(lib.ntb200_matmult_batch(L.F32, arr(da, order), arr(db, order), arr(dc, order), 5, 40, 24, 24, 56, 0, 0, s))
    assert np.array_equal(host(dc), exp)


def test_host_buffer_entry_point(api, oracle):
    """ntb200_matmult_host: the reference's CPU-pointer contract, staged through the device."""
    rng = np.random.default_rng(47)
    a, b = normal(rng, (9, 64, 48), np.float16, 0.5), normal(rng, (9, 80, 48), np.float16, 0.5)
    c = np.zeros((9, 64, 80), np.float16)
    api.matmult_host(a, b, c, False, True)
    assert oracle.rel_fro(c, oracle.matmult(a, b, False, True)) <= F16_TOL
    a2, b2 = normal(rng, (1500, 70), np.float32), normal(rng, (70, 90), np.float32)
    c2 = normal(rng, (1500, 90), np.float32)
    exp = c2.copy()
    oracle.matmult_into(a2, b2, exp)
    api.matmult_host(a2, b2, c2)
    assert np.array_equal(c2, exp)


def test_empty_and_k_zero(api):
    z = api.matmult(torch.zeros((0, 5), device="cuda"), torch.ones((5, 3), device="cuda"))
    assert z.shape == (0, 3)
    r = api.matmult(torch.ones((4, 0), device="cuda"), torch.ones((0, 3), device="cuda"))
    assert torch.equal(r, torch.zeros((4, 3), device="cuda"))


def test_errors_match_the_reference(api):
    a = torch.zeros((4, 5), device="cuda")
    with pytest.raises(ValueError, match="Expected second tensor rows"):
        api.matmult(a, torch.zeros((4, 5), device="cuda"))
    with pytest.raises(ValueError, match="same dtype"):
        api.matmult(a, torch.zeros((5, 5), device="cuda", dtype=torch.float16))
    with pytest.raises(ValueError, match="number type"):
        api.matmult(a.bool(), a.bool().t())
    with pytest.raises(ValueError, match="contiguous"):
        api.matmult(a, a.t(), out=torch.zeros((4, 8), device="cuda")[:, ::2])


def test_launches_are_counted_and_status_is_clean(api, L):
    before = L.launch_count()
    api.matmult(torch.ones((128, 64), device="cuda", dtype=torch.float16),
                torch.ones((64, 128), device="cuda", dtype=torch.float16))
    assert L.launch_count() == before + 1
    L.check(L.lib().ntb200_check_device_status(None))


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n", [(131, 77, 65), (256, 512, 384), (1024, 2048, 1280)])
def test_int32_on_tensor_cores_bit_exact(api, oracle, L, ta, tb, m, k, n):
    """Int32 as ten products of 8-bit limbs on kind::i8: full-range operands, wrap modulo 2^32, any strides."""
    rng = np.random.default_rng(61 + m)
    info = np.iinfo(np.int32)
    a, b = operands(rng, m, k, n, ta, tb, np.int32, ints=(info.min, info.max))
    got = host(api.matmult(dev(a), dev(b), ta, tb, route=L.ROUTE_TENSOR))
    assert L.last_route() == "umma_i32_limbs"
    assert np.array_equal(got, oracle.matmult(a, b, ta, tb))


def test_int32_tensor_route_accumulate_bias_batch(api, oracle, L):
    rng = np.random.default_rng(67)
    a, w = integers(rng, (3, 200, 96), np.int32, -10 ** 9, 10 ** 9), integers(rng, (96, 136), np.int32, -10 ** 9, 10 ** 9)
    bias, c0 = integers(rng, (136,), np.int32, -10 ** 9, 10 ** 9), integers(rng, (3, 200, 136), np.int32, -10 ** 9, 10 ** 9)
    got = host(api.linear(dev(a), dev(w), dev(bias), route=L.ROUTE_TENSOR))
    assert L.last_route() == "umma_i32_limbs"
    assert np.array_equal(got, oracle.linear(a, w, bias))
    out = dev(c0)
    api.matmult(dev(a), dev(w), out=out, route=L.ROUTE_TENSOR)
    exp = c0.copy()
    for i in range(3):
        oracle.matmult_into(a[i], w, exp[i])
    assert np.array_equal(host(out), exp)


@pytest.mark.parametrize("ta,tb", FLAGS)
@pytest.mark.parametrize("m,k,n,dtype", [(136, 72, 64, np.int16), (256, 520, 384, np.uint16), (1024, 9000, 1280, np.int16)])
def test_int16_on_tensor_cores_bit_exact(api, oracle, L, ta, tb, m, k, n, dtype):
    """Int16 / UInt16 as three products of 8-bit limbs on kind::i8 (two GEMMs per 8192-wide K chunk): full-range
    operands, wrap modulo 2^16, all transpose combinations; K = 9000 crosses a chunk boundary."""
    rng = np.random.default_rng(73 + m)
    info = np.iinfo(dtype)
    a, b = operands(rng, m, k, n, ta, tb, dtype, ints=(info.min, info.max))
    # numpy has no 16-bit cuda tensors for uint16 in torch: travel as int16 bit patterns
    da, db = torch.from_numpy(a.view(np.int16)).cuda(), torch.from_numpy(b.view(np.int16)).cuda()
    got = host(api.matmult(da, db, ta, tb, route=L.ROUTE_TENSOR)).view(dtype)
    assert L.last_route() == "umma_i16_limbs"
    assert np.array_equal(got, oracle.matmult(a.view(np.int16), b.view(np.int16), ta, tb).view(dtype))


def test_int16_tensor_route_accumulate_bias_batch(api, oracle, L):
    rng = np.random.default_rng(79)
    a, w = integers(rng, (3, 200, 96), np.int16, -32768, 32767), integers(rng, (96, 136), np.int16, -32768, 32767)
    bias, c0 = integers(rng, (136,), np.int16, -32768, 32767), integers(rng, (3, 200, 136), np.int16, -32768, 32767)
    got = host(api.linear(dev(a), dev(w), dev(bias), route=L.ROUTE_TENSOR))
    assert L.last_route() == "umma_i16_limbs"
    assert np.array_equal(got, oracle.linear(a, w, bias))
    out = dev(c0)
    api.matmult(dev(a), dev(w), out=out, route=L.ROUTE_TENSOR)
    exp = c0.copy()
    for i in range(3):
        oracle.matmult_into(a[i], w, exp[i])
    assert np.array_equal(host(out), exp)
    # large problems take the limb route by themselves
    big_a, big_b = integers(rng, (512, 1024), np.int16, -32768, 32767), integers(rng, (1024, 512), np.int16, -32768, 32767)
    got = host(api.matmult(dev(big_a), dev(big_b)))
    assert L.last_route() == "umma_i16_limbs"
    assert np.array_equal(got, oracle.matmult(big_a, big_b))


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("weights_nk", [False, True])
def test_few_rows_stream_the_weights(api, oracle, L, m, weights_nk, bf16):
    """One or two rows of 16-bit floats against a large weight matrix take the CUDA-core streaming kernels
    (weights [K, N] or a transposed view of weights [N, K]); fp32 accumulation, one rounding, optional bias and C +=."""
    rng = np.random.default_rng(89 + m)
    k, n = 1544, 1160                                   # ragged against the 128 / 2048 K slabs and the column blocks
    x32, w32 = normal(rng, (m, k), np.float32, 0.5), normal(rng, (k, n), np.float32, 0.5)
    b32, c32 = normal(rng, (n,), np.float32), normal(rng, (m, n), np.float32)
    cd = Codec(oracle, bf16)
    x, bias = cd.enc(x32), cd.enc(b32)
    w = cd.enc(np.ascontiguousarray(w32.T)).t() if weights_nk else cd.enc(w32)    # [K, N] view either way
    got = api.linear(x, w, bias)
    assert L.last_route() == "gemv_simt"
    check_16bit(oracle, cd, cd.dec(got), x32, w32, b32, what="weight streaming, bias")
    out = cd.enc(c32)
    api.matmult(x, w, out=out)                           # C += x . w
    assert L.last_route() == "gemv_simt"
    check_16bit(oracle, cd, cd.dec(out), x32, w32, c32, what="weight streaming, C +=")
    # an explicit route request is honoured, and three rows are the tensor cores' again
    api.matmult(x, w, route=L.ROUTE_TENSOR)
    assert L.last_route().startswith(("umma_f16", "umma_bf16"))
    api.matmult(x[:1].repeat(3, 1), w)
    assert L.last_route().startswith(("umma_f16", "umma_bf16"))


@pytest.mark.gpu
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("m,n,k,weights_nk", [(3, 4096, 4096, False), (16, 4100, 4096, True), (100, 4096, 8192, False),
                                              (128, 8192, 4096, True), (256, 2048, 8192, False), (300, 2048, 8192, True),
                                              (512, 4096, 4096, False),     # two pairs per tile (S = 2)
                                              (300, 2052, 8192, True),      # rows of C not 16-byte aligned: no TMA store, copy-out pass
                                              (260, 2050, 4096, True)])     # rows of C not 8-byte aligned: scalar stores
def test_few_rows_split_the_k_axis(api, oracle, L, m, n, k, weights_nk, bf16):
    """A few rows (or a few hundred against a deep, narrow weight matrix) of 16-bit floats: K is cut into slices that run
    side by side as fp32 partial tiles, and a second kernel adds them, the bias and the previous C and rounds once."""
    rng = np.random.default_rng(97 + m)
    x32, w32 = normal(rng, (m, k), np.float32, 0.5), normal(rng, (k, n), np.float32, 0.5)
    b32, c32 = normal(rng, (n,), np.float32), normal(rng, (m, n), np.float32)
    cd = Codec(oracle, bf16)
    x, bias = cd.enc(x32), cd.enc(b32)
    w = cd.enc(np.ascontiguousarray(w32.T)).t() if weights_nk else cd.enc(w32)    # [K, N] view either way
    dec = cd.dec
    # up to 128 rows the K slices run inside a thread-block cluster (one launch, partial tiles added through
    # distributed shared memory); more rows take the K slices as batches of the pair kernel plus a reduction kernel
    base = "umma_bf16" if bf16 else "umma_f16"
    # up to 128 rows: S CTAs of a cluster per 128-row tile; more rows: S CTA pairs of a cluster per 256 x 256 tile, or
    # (when the clusters would not fit in one wave) K slices as batches of the pair kernel plus a reduction kernel
    split_routes = (base + "_clusterk",) if m <= 128 else (base + "_pairclusterk", base + "_splitk")
    got = api.linear(x, w, bias)
    assert L.last_route() in split_routes
    # K = 4096 / 8192: Float16 is beyond the depth at which fp32 accumulation stays within 2e-3 of the reference's
    # per-16-k rounding; both distances are measured and reported, the bar is on the fp32-accumulate value
    check_16bit(oracle, cd, dec(got), x32, w32, b32, what="K slices, bias")
    out = cd.enc(c32)
    api.matmult(x, w, out=out)                           # C += x . w
    assert L.last_route() in split_routes
    check_16bit(oracle, cd, dec(out), x32, w32, c32, what="K slices, C +=")
    # the left half of the columns on its own (a strided view, possibly too small to split) gives the same sums up to
    # the order of the fp32 additions
    half = api.matmult(x, w[:, : n // 2])
    both = api.matmult(x, w)
    assert L.last_route() in split_routes
    assert oracle.rel_fro(dec(both)[:, : n // 2], dec(half)) <= 1e-3


@pytest.mark.gpu
def test_pair_cluster_exchange_variants_agree_bit_for_bit():
    """The K slices of a pair cluster are summed in slice order whichever way the partial tiles travel (L2 scratch and
    TMA stores, L2 scratch and the copy-out pass, distributed shared memory): the three give identical bits.  The
    switches are read once per process, so each variant runs in a process of its own."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    code = (
        "import sys, torch, hashlib\n"
        "sys.path.insert(0, %r)\n"
        "from neurotensor_b200 import _lib, api\n"
        "g = torch.Generator(device='cuda').manual_seed(5)\n"
        "out = []\n"
        "for (m, k, n) in ((512, 4096, 4096), (300, 8192, 2048)):\n"
        "    a = (torch.randn((m, k), generator=g, device='cuda') * 0.5).half()\n"
        "    b = (torch.randn((k, n), generator=g, device='cuda') * 0.5).half()\n"
        "    bias = torch.randn((n,), generator=g, device='cuda').half()\n"
        "    c = api.linear(a, b, bias)\n"
        "    assert _lib.last_route() == 'umma_f16_pairclusterk', _lib.last_route()\n"
        "    out.append(hashlib.sha256(c.cpu().numpy().tobytes()).hexdigest())\n"
        "print(' '.join(out))\n" % ROOT)
    digests = {}
    for name, env in (("l2+tma", {}), ("l2+copy-out", {"NTB200_PAIR_CLUSTER_COPY_OUT": "1"}), ("dsmem", {"NTB200_PAIR_CLUSTER_DSMEM": "1"})):
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=dict(os.environ, **env))
        assert r.returncode == 0, name + ": " + r.stderr[-2000:]
        digests[name] = r.stdout.strip().splitlines()[-1]
    assert len(set(digests.values())) == 1, digests


def test_pinned_host_buffers_from_the_library(api, oracle, L):
    """ntb200_host_alloc / ntb200_host_register give page-locked host memory for ntb200_matmult_host."""
    import ctypes
    lib = L.lib()
    rng = np.random.default_rng(71)
    shape_a, shape_b, shape_c = (4, 96, 64), (4, 64, 80), (4, 96, 80)
    bufs = []
    for shape in (shape_a, shape_b, shape_c):
        p = ctypes.c_void_p()
        L.check(lib.ntb200_host_alloc(ctypes.byref(p), int(np.prod(shape)) * 4))
        arr = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_float)), shape=shape)
        bufs.append((p, arr))
    (pa, a), (pb, b), (pc, c) = bufs
    a[...] = normal(rng, shape_a, np.float32)
    b[...] = normal(rng, shape_b, np.float32)
    c[...] = 0
    api.matmult_host(a, b, c, accumulate=False)
    assert np.array_equal(c, oracle.matmult(a.copy(), b.copy()))
    for p, _ in bufs:
        L.check(lib.ntb200_host_free(p))
    own = np.zeros((64, 64), np.float32)
    L.check(lib.ntb200_host_register(own.ctypes.data, own.nbytes))
    L.check(lib.ntb200_host_unregister(own.ctypes.data))


@pytest.mark.gpu
@pytest.mark.parametrize("a_shape,b_shape,ta,tb", [
    ((5, 2, 3, 4), (5, 2, 4, 3), False, False),      # "matmult tensors (no bigger)", tests/src/matmult_test.cpp:108-120
    ((5, 2, 4, 3), (5, 2, 4, 3), True, False),       # "matmult tensors Ta", :142-153
    ((5, 2, 4, 3), (5, 2, 4, 3), False, True),       # "matmult tensors Tb", :154-165
    ((5, 2, 4, 3), (5, 4, 3), True, False),          # "Ta (bigger a)", :167-178
    ((5, 2, 4, 3), (5, 4, 3), False, True),          # "Tb (bigger a)", :179-190
    ((5, 3, 4), (5, 2, 4, 3), False, False),         # the items of b carry the batch dimension
])
@pytest.mark.parametrize("scattered", [False, True])
def test_tensor_of_tensors_matmult(api, oracle, L, a_shape, b_shape, ta, tb, scattered):
    """Tensor-of-tensors operands: item i of the result equals matmult(a[i], b[i]), bit for bit (the reference's own
    check, `all(o1 == o[i])`), for lists split from one tensor (equally spaced pointers, one strided launch) and for
    lists of separately allocated tensors in shuffled order (device pointer tables)."""
    rng = np.random.default_rng(101)
    a = rng.integers(0, 3, a_shape).astype(np.float32) + normal(rng, a_shape, np.float32, 0.25)
    b = rng.integers(0, 3, b_shape).astype(np.float32) + normal(rng, b_shape, np.float32, 0.25)
    if scattered:
        order = [3, 0, 4, 1, 2]
        a_list = [dev(a[i].copy()) for i in order]
        b_list = [dev(b[i].copy()) for i in order]
        a, b = a[order], b[order]
    else:
        da, db = dev(a), dev(b)
        a_list, b_list = [da[i] for i in range(5)], [db[i] for i in range(5)]
    out = api.matmult_tensors(a_list, b_list, ta, tb)
    assert len(out) == 5
    for i in range(5):
        single = api.matmult(a_list[i], b_list[i], ta, tb)
        assert torch.equal(out[i], single), "item %d differs from the 2-operand call" % i
        ai = np.swapaxes(a[i], -1, -2) if ta else a[i]
        bi = np.swapaxes(b[i], -1, -2) if tb else b[i]
        assert np.array_equal(host(out[i]), oracle.matmult(ai, bi))


@pytest.mark.gpu
def test_tensor_of_tensors_errors(api):
    x = torch.zeros((2, 3, 4), device="cuda")
    with pytest.raises(ValueError, match="same number of sub-tensors"):
        api.matmult_tensors([x, x], [x])
    with pytest.raises(ValueError, match="same shape"):
        api.matmult_tensors([x, x[:, :2]], [x, x])
    with pytest.raises(ValueError, match="same dtype"):
        api.matmult_tensors([x, x], [x.half(), x.half()], False, True)
    with pytest.raises(ValueError, match="Expected second tensor rows to be 4 when it was 3"):
        api.matmult_tensors([x], [x])


@pytest.mark.gpu
def test_hodge_laplacian_products(api, oracle):
    """The two matmult calls of the TDA Hodge Laplacian on signed boundary matrices (entries -1, 0, 1 scaled by radii):
    B_{k+1} B_{k+1}^T + B_k^T B_k, Float32, bit-exact against the oracle's chains and one fp32 add."""
    rng = np.random.default_rng(103)
    bk = (rng.integers(-1, 2, (21, 35)) * rng.uniform(0.5, 1.5, (21, 35))).astype(np.float32)      # [k-1 simplices, k simplices]
    bkp1 = (rng.integers(-1, 2, (35, 40)) * rng.uniform(0.5, 1.5, (35, 40))).astype(np.float32)    # [k simplices, k+1 simplices]
    got = api.hodge_laplacian_from_boundaries(dev(bkp1), dev(bk))
    exp = oracle.matmult(bkp1, bkp1.T.copy()) + oracle.matmult(bk.T.copy(), bk)
    assert np.array_equal(host(got), exp.astype(np.float32))
    assert np.array_equal(host(api.hodge_laplacian_from_boundaries(dev(bkp1))), oracle.matmult(bkp1, bkp1.T.copy()))


@pytest.mark.gpu
@pytest.mark.parametrize("np_dtype", [np.complex64, np.complex128])
def test_complex_matmult_is_the_references_lanewise_product(api, oracle, L, np_dtype):
    """Complex64 / Complex128: the reference's SIMD traits multiply the interleaved (re, im) lanes independently, so its
    matmult gives C.re = A.re B.re and C.im = A.im B.im as two exact FMA chains; the CUDA-core route reproduces that bit
    for bit (2-D, batched with a lower-rank operand, transposed views, C +=), and a tensor-core request is refused."""
    rng = np.random.default_rng(107)
    fdt = np.float32 if np_dtype == np.complex64 else np.float64
    cplx = lambda shape: (normal(rng, shape, fdt) + 1j * normal(rng, shape, fdt)).astype(np_dtype)
    a, b = cplx((3, 70, 45)), cplx((45, 133))
    got = api.matmult(dev(a), dev(b))
    assert L.last_route() == "simt"
    exp = oracle.matmult(a, b)
    assert np.array_equal(host(got), exp)
    assert not np.allclose(exp, a @ b)                   # not the mathematical product
    assert np.array_equal(exp.real, oracle.matmult(np.ascontiguousarray(a.real), np.ascontiguousarray(b.real)))
    bt = cplx((133, 45))
    got_t = api.matmult(dev(a), dev(bt), transpose_b=True)
    assert np.array_equal(host(got_t), oracle.matmult(a, bt, transpose_b=True))
    at = cplx((3, 45, 70))
    assert np.array_equal(host(api.matmult(dev(at), dev(b), transpose_a=True)), oracle.matmult(at, b, transpose_a=True))
    # C += : the chains continue from the previous contents, lane by lane
    c0 = cplx((70, 133))
    out = dev(c0.copy())
    api.matmult(dev(a[0]), dev(b), out=out)
    exp_re = oracle.matmult_into(np.ascontiguousarray(a[0].real), np.ascontiguousarray(b.real), np.ascontiguousarray(c0.real))
    exp_im = oracle.matmult_into(np.ascontiguousarray(a[0].imag), np.ascontiguousarray(b.imag), np.ascontiguousarray(c0.imag))
    assert np.array_equal(host(out).real, exp_re) and np.array_equal(host(out).imag, exp_im)
    with pytest.raises(L.Ntb200Error):
        api.matmult(dev(a), dev(b), route=L.ROUTE_TENSOR)


def test_complex32_matmult(api, oracle, L):
    """Complex32 (pairs of Float16): lane-wise like Complex64, the running sums rounded to Float16 at the edges of the
    reference's K tile for this type, every 8 k-steps.  Bit for bit against the oracle (which is pinned on the compiled
    reference kernel for this type): 2-D, batched against a 2-D operand, both transposed views, C +=."""
    rng = np.random.default_rng(109)
    pairs = lambda shape: normal(rng, shape + (2,), np.float16, 0.5)
    as_c32 = lambda arr: torch.view_as_complex(torch.from_numpy(arr).cuda())
    back = lambda t: torch.view_as_real(t).cpu().numpy()
    a, b = pairs((3, 70, 45)), pairs((45, 133))
    got = api.matmult(as_c32(a), as_c32(b))
    assert L.last_route() == "simt" and got.dtype == torch.complex32
    assert np.array_equal(back(got), oracle.matmult_complex32(a, b))
    bt, at = pairs((133, 45)), pairs((3, 45, 70))
    assert np.array_equal(back(api.matmult(as_c32(a), as_c32(bt), transpose_b=True)), oracle.matmult_complex32(a, bt, transpose_b=True))
    assert np.array_equal(back(api.matmult(as_c32(at), as_c32(b), transpose_a=True)), oracle.matmult_complex32(at, b, transpose_a=True))
    # fp32 lanes rounded once would differ: the tile-edge rounding is really there
    once = np.stack([(a[0, ..., i].astype(np.float32) @ b[..., i].astype(np.float32)).astype(np.float16) for i in (0, 1)], axis=-1)
    assert not np.array_equal(back(got)[0], once)
    c0 = pairs((70, 133))
    out = as_c32(c0.copy())
    api.matmult(as_c32(a[0]), as_c32(b), out=out)
    exp = np.stack([oracle.matmult_into(np.ascontiguousarray(a[0, ..., i]), np.ascontiguousarray(b[..., i]), np.ascontiguousarray(c0[..., i]),
                                        bf16="c32-lane") for i in (0, 1)], axis=-1)
    assert np.array_equal(back(out), exp)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["f16", "bf16", "i8"])
@pytest.mark.parametrize("m,n,k", [(300, 528, 48), (256, 512, 384), (515, 272, 144)])
def test_shallow_k_takes_the_wide_epilogue(api, oracle, L, kind, m, n, k):
    """At most six K blocks on CTA pairs: two epilogue warps per lane quadrant share a tile's 256 columns.  Ragged edges,
    bias, C += and 8-bit outputs go through the same staging and TMA stores as the four-warp epilogue."""
    rng = np.random.default_rng(113 + m)
    if kind == "i8":
        a, b = integers(rng, (m, k), np.int8, -128, 127), integers(rng, (k, n), np.int8, -128, 127)
        c0 = integers(rng, (m, n), np.int8, -128, 127)
        got = api.matmult(dev(a), dev(b))
        assert L.last_route() == "umma_i8"
        assert np.array_equal(host(got), oracle.matmult(a, b))
        out = dev(c0.copy())
        api.matmult(dev(a), dev(b), out=out)
        assert np.array_equal(host(out), oracle.matmult_into(a, b, c0.copy()))
        return
    bf16 = kind == "bf16"
    a32, b32 = normal(rng, (m, k), np.float32, 0.5), normal(rng, (k, n), np.float32, 0.5)
    bias32, c32 = normal(rng, (n,), np.float32), normal(rng, (m, n), np.float32)
    cd = Codec(oracle, bf16)
    got = api.linear(cd.enc(a32), cd.enc(b32), cd.enc(bias32))
    assert L.last_route().startswith(("umma_f16", "umma_bf16"))
    check_16bit(oracle, cd, cd.dec(got), a32, b32, bias32, what="shallow K, bias")
    out = cd.enc(c32)
    api.matmult(cd.enc(a32), cd.enc(b32), out=out)
    check_16bit(oracle, cd, cd.dec(out), a32, b32, c32, what="shallow K, C +=")
    bt = cd.enc(np.ascontiguousarray(b32.T)).t()            # K-major B
    check_16bit(oracle, cd, cd.dec(api.matmult(cd.enc(a32), bt)), a32, b32, what="shallow K, K-major B")
