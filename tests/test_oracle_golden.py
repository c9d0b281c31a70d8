"""Pins the CPU oracle against the reference's own committed golden vectors (Float32) and checks the
semantics it restates for the dtypes the reference's tests do not cover.

Reference tests mirrored: tests/src/linear_autograd_test.cpp:128-196, tests/src/conv_autograd_test.cpp:249-374,
tests/src/col_im_autograd_test.cpp:77-116, tests/src/matmult_test.cpp:10-189; all compare with
allclose(rtol=1e-5, atol=1e-8) (nt/functional/tensor_files/compare.h:34).
"""
import os

import numpy as np
import pytest

from conftest import REF_GOLDEN

RTOL, ATOL = 1e-5, 1e-8


def g(name):
    return np.load(os.path.join(REF_GOLDEN, name + ".npy"))


def close(a, b):
    return np.allclose(a, b, rtol=RTOL, atol=ATOL)


def test_linear_golden(oracle):
    x, w, b, grad = g("linear_input"), g("linear_weight"), g("linear_bias"), g("linear_grad")
    out = oracle.linear(x, w, b, transpose_b=True)
    assert close(out, x @ w.T + b)
    dx, dw = oracle.matmult_backward(x, w, grad, False, True)
    assert close(dx, g("linear_xgrad"))
    # the 2-D weight was repeated over the batch; its gradient is reduced back to the weight's shape
    assert close(dw.sum(axis=0), g("linear_wgrad"))
    assert close(grad.sum(axis=(0, 1)), g("linear_bgrad"))


def test_linear_complex_golden(oracle):
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))
    grad = g("linear_complex_grad")
    for xs, ws, bs, xg, wg, bg in (("input_a", "weight", "bias", "x1grad", "wgrad", "bgrad"),
                                   ("input_b", "weight2", "bias2", "x2grad", "w2grad", "b2grad")):
        x, w, b = g("linear_complex_" + xs), g("linear_complex_" + ws), g("linear_complex_" + bs)
        o = oracle.linear(x, w, b, transpose_b=True)
        s = sig(o.astype(np.float64))
        go = (grad * s * (1 - s)).astype(np.float32)
        dx, dw = oracle.matmult_backward(x, w, go, False, True)
        assert close(dx, g("linear_complex_" + xg))
        assert close(dw.sum(axis=0), g("linear_complex_" + wg))
        assert close(go.sum(axis=(0, 1)), g("linear_complex_" + bg))


@pytest.mark.parametrize("ext", ["", "_batched"])
def test_conv2d_golden(oracle, ext):
    x, w = g("conv2d_input" + ext), g("conv2d_weight" + ext)
    out = oracle.conv2d(x, w, stride=1, padding=1)
    assert out.shape == g("conv2d_output" + ext).shape
    assert close(out, g("conv2d_output" + ext))
    dx, dw = oracle.conv2d_backward(x, w, g("conv2d_grad" + ext), stride=1, padding=1)
    assert close(dx, g("conv2d_xgrad" + ext))
    assert close(dw, g("conv2d_wgrad" + ext))


def test_unfold2d_golden(oracle):
    x = g("unfold_input")
    col = oracle.unfold2d(x, (3, 2), dilation=(1, 2), padding=1, stride=(2, 2))
    assert np.array_equal(col, g("unfold_output"))
    dx = oracle.unfold2d_backward(g("unfold_grad"), x.shape[-2:], (3, 2), dilation=(1, 2), padding=1, stride=(2, 2))
    assert close(dx.reshape(x.shape), g("unfold_input_grad"))


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_matmult_shapes_and_flags(oracle, ta, tb):
    """Shape contract of tests/src/matmult_test.cpp:10-107 (all four flag combinations, 2-D and 3-D)."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((5, 7) if ta else (7, 5)).astype(np.float32)
    b = rng.standard_normal((3, 5) if tb else (5, 3)).astype(np.float32)
    out = oracle.matmult(a, b, ta, tb)
    ref = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    assert out.shape == (7, 3) and np.allclose(out, ref, rtol=RTOL, atol=ATOL)
    a3 = np.stack([a, 2 * a])
    out3 = oracle.matmult(a3, b, ta, tb)       # lower-rank operand repeated over the batch
    assert out3.shape == (2, 7, 3) and np.array_equal(out3[0], out)
    with pytest.raises(ValueError):
        oracle.matmult(a, b, not ta, tb)


def test_float32_is_one_fma_chain(oracle):
    """Each output is a single ascending-k fused-multiply-add chain in fp32 (simde_traits_avx2.h:250-256)."""
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 37)).astype(np.float32)
    b = rng.standard_normal((37, 5)).astype(np.float32)
    out = oracle.matmult(a, b)
    exp = np.zeros((3, 5), np.float32)
    for i in range(3):
        for j in range(5):
            acc = np.float64(0)
            accf = np.float32(0)
            for k in range(37):
                # fma: exact product + accumulator, rounded once (float64 holds a*b+acc of float32s exactly enough)
                accf = np.float32(np.float64(a[i, k]) * np.float64(b[k, j]) + np.float64(accf))
            exp[i, j] = accf
    assert np.array_equal(out, exp)


def test_float16_rounds_every_16_k(oracle):
    """fp32 chain inside a 16-wide K tile, running sum rounded to fp16 at each tile edge
    (simde_traits_avx2.h:1133-1135,1160-1165,1230-1236 + nt_matmult.hpp:196)."""
    rng = np.random.default_rng(2)
    a = (rng.standard_normal((4, 70)) * 0.5).astype(np.float16)
    b = (rng.standard_normal((70, 6)) * 0.5).astype(np.float16)
    out = oracle.matmult(a, b)
    exp = np.zeros((4, 6), np.float16)
    for i in range(4):
        for j in range(6):
            c = np.float16(0)
            for k0 in range(0, 70, 16):
                acc = np.float32(c)
                for k in range(k0, min(k0 + 16, 70)):
                    acc = np.float32(np.float64(np.float32(a[i, k])) * np.float64(np.float32(b[k, j])) + np.float64(acc))
                c = np.float16(acc)
            exp[i, j] = c
    assert np.array_equal(out.view(np.uint16), exp.view(np.uint16))
    # and it differs from a round-once fp32 accumulation, which is what the tolerance has to absorb
    once = (a.astype(np.float32) @ b.astype(np.float32)).astype(np.float16)
    assert oracle.rel_fro(out, once) < 2e-3


@pytest.mark.parametrize("dt", [np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32])
def test_integers_wrap_in_their_own_width(oracle, dt):
    rng = np.random.default_rng(3)
    info = np.iinfo(dt)
    a = rng.integers(info.min, info.max, size=(9, 33), endpoint=True).astype(dt)
    b = rng.integers(info.min, info.max, size=(33, 11), endpoint=True).astype(dt)
    out = oracle.matmult(a, b)
    exact = np.array([[sum(int(a[i, k]) * int(b[k, j]) for k in range(33)) for j in range(11)] for i in range(9)],
                     dtype=object)
    bits = info.bits
    wrapped = np.array([[int(v) % (1 << bits) for v in row] for row in exact], dtype=object)
    got = np.array([[int(v) % (1 << bits) for v in row] for row in out.astype(object)], dtype=object)
    assert out.dtype == dt and (wrapped == got).all()


def test_out_variant_accumulates(oracle):
    """matmult(a, b, out) computes out += a.b (matmult_cpu.cpp:137-153)."""
    rng = np.random.default_rng(4)
    a = rng.integers(-5, 5, (6, 8)).astype(np.int32)
    b = rng.integers(-5, 5, (8, 4)).astype(np.int32)
    c = rng.integers(-5, 5, (6, 4)).astype(np.int32)
    exp = c + a @ b
    oracle.matmult_into(a, b, c)
    assert np.array_equal(c, exp)


def test_bf16_is_fp32_chain_on_widened_inputs(oracle):
    rng = np.random.default_rng(5)
    a32 = rng.standard_normal((8, 40)).astype(np.float32)
    b32 = rng.standard_normal((40, 8)).astype(np.float32)
    a, b = oracle.bf16_round(a32), oracle.bf16_round(b32)
    out = oracle.matmult(a, b, bf16=True)
    ref = oracle.matmult(oracle.bf16_widen(a), oracle.bf16_widen(b))
    assert np.array_equal(out, oracle.bf16_round(ref))


def test_empty_and_ragged(oracle):
    a = np.zeros((0, 5), np.float32)
    b = np.ones((5, 3), np.float32)
    assert oracle.matmult(a, b).shape == (0, 3)
    assert np.array_equal(oracle.matmult(np.ones((2, 0), np.float32), np.ones((0, 3), np.float32)), np.zeros((2, 3)))
    rng = np.random.default_rng(6)
    for m, k, n in [(1, 1, 1), (17, 1, 31), (33, 130, 19), (129, 47, 65)]:
        a = rng.integers(-3, 3, (m, k)).astype(np.float32)
        b = rng.integers(-3, 3, (k, n)).astype(np.float32)
        assert np.array_equal(oracle.matmult(a, b), a @ b)


def test_complex_matmult_follows_the_simd_traits_lanes():
    """The reference's complex GEMM traits are the float / double lane operations on interleaved (re, im) data
    (simde_traits_avx2.h:915-1000, 1029-1110), so matmult gives re x re and im x im as independent real chains."""
    from oracle import oracle
    rng = np.random.default_rng(5)
    for cdt, fdt in ((np.complex64, np.float32), (np.complex128, np.float64)):
        a = (rng.standard_normal((2, 9, 21)) + 1j * rng.standard_normal((2, 9, 21))).astype(cdt)
        b = (rng.standard_normal((21, 13)) + 1j * rng.standard_normal((21, 13))).astype(cdt)
        got = oracle.matmult(a, b)
        assert got.dtype == cdt and got.shape == (2, 9, 13)
        assert np.array_equal(got.real, oracle.matmult(np.ascontiguousarray(a.real), np.ascontiguousarray(b.real)))
        assert np.array_equal(got.imag, oracle.matmult(np.ascontiguousarray(a.imag), np.ascontiguousarray(b.imag)))
        assert got.real.dtype == fdt
        assert not np.allclose(got, a @ b)
