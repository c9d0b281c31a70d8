"""optimizers::SGD::step and optimizers::Adam::step (nt/nn/Optimizers.cpp:8-17, 68-98).

The oracle repeats the reference's whole-tensor operations in the parameter's dtype; the CPU tests pin it against
scalar restatements of the same source lines, the GPU tests compare ntb200_sgd_step / ntb200_adam_step with it
bit for bit for Float32, Float16 and BFloat16 (which the reference does not have: same sequence, bf16 roundings)."""
import math

import numpy as np
import pytest


def _inputs(seed, n, dtype):
    rng = np.random.default_rng(seed)
    p = rng.standard_normal(n).astype(dtype)
    g = (rng.standard_normal(n) * 3).astype(dtype)
    k = min(n, 4)
    g[:k] = np.array([25.0, -30.0, 0.0, 1e-3], dtype=dtype)[:k]    # clipped both ways, zero, tiny
    m = (rng.standard_normal(n) * 0.1).astype(dtype)
    v = np.abs(rng.standard_normal(n) * 0.01).astype(dtype)
    return p, g, m, v


def test_oracle_sgd_is_the_source_formula(oracle):
    p, g, _, _ = _inputs(1, 64, np.float32)
    got = oracle.sgd_step(p, g, lr=0.01)
    for i in range(64):
        gi = np.float32(min(max(float(g[i]), -10.0), 10.0)) * np.float32(0.01)      # clip_, then *= lr, in float
        assert got[i] == np.float32(p[i] - np.float32(gi))


def test_oracle_adam_is_the_source_formula(oracle):
    """Scalar walk through Optimizers.cpp:82-95 in float32, one element at a time."""
    p, g, m, v = _inputs(2, 64, np.float32)
    f = np.float32
    b1, b2, lr, eps, t = 0.9, 0.999, 0.001, 1e-8, 0
    got_p, got_m, got_v = oracle.adam_step(p, g, m, v, lr, b1, b2, eps, t)
    for i in range(64):
        mi = f(f(f(m[i] * f(b1)) + f(1 - b1)) * g[i])
        vi = f(f(f(v[i] * f(b2)) + f(1 - b2)) * f(g[i] * g[i]))
        m_hat = f(mi / f((1 - b1) ** t))
        v_hat = f(vi / f((1 - b2) ** t))
        with np.errstate(divide="ignore", invalid="ignore"):
            u = f(f(f(lr) * m_hat) / f(f(np.sqrt(v_hat)) + f(eps)))
        u = min(max(u, f(-10)), f(10))
        exp = f(p[i] - u)
        assert got_m[i] == mi and got_v[i] == vi
        assert got_p[i] == exp or (math.isnan(float(exp)) and math.isnan(float(got_p[i])))
    # from zero moments the first update is lr * (1-b1) g / (sqrt((1-b2) g^2) + eps): sign(g) * lr * 0.1 / sqrt(0.001)
    z = np.zeros(8, np.float32)
    gg = np.array([0.5, -2.0, 3.0, -0.25, 1.0, 7.0, -9.0, 4.0], np.float32)
    new_p, _, _ = oracle.adam_step(z.copy(), gg, z.copy(), z.copy())
    assert np.allclose(new_p, -np.sign(gg) * 0.001 * 0.1 / math.sqrt(0.001), rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("n", [1, 1000, 2 ** 20 + 3])   # one element; one block; more than one grid pass
def test_sgd_step_bit_exact(oracle, dtype, n):
    from gpu_util import dev, host
    from neurotensor_b200 import api
    p, g, _, _ = _inputs(3 + n, n, dtype)
    pd = dev(p)
    api.sgd_step(pd, dev(g), lr=0.05)
    assert np.array_equal(host(pd), oracle.sgd_step(p, g, lr=0.05))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("t", [0, 3])
def test_adam_step_bit_exact_over_three_steps(oracle, dtype, t):
    from gpu_util import dev, host
    from neurotensor_b200 import api
    n = 2 ** 18 + 5
    p, g, m, v = _inputs(7 + t, n, dtype)
    if dtype == np.float16:
        g[2] = 1.0      # epsilon underflows to 0 in Float16, so a zero gradient is 0/0 there as in the reference
    pd, md, vd = dev(p), dev(m), dev(v)
    for step in range(3):
        gs = (g * dtype(1.0 + 0.25 * step)).astype(dtype)
        api.adam_step(pd, dev(gs), md, vd, lr=0.01, beta1=0.9, beta2=0.999, epsilon=1e-8, t=t)
        p, m, v = oracle.adam_step(p, gs, m, v, lr=0.01, beta1=0.9, beta2=0.999, epsilon=1e-8, t=t)
        assert np.array_equal(host(md), m)
        assert np.array_equal(host(vd), v)
        assert np.array_equal(host(pd), p, equal_nan=True)


@pytest.mark.gpu
def test_optimizer_steps_bf16_and_errors(oracle):
    import torch
    from gpu_util import dev, host
    from neurotensor_b200 import _lib, api
    p, g, m, v = (oracle.bf16_round(x) for x in _inputs(11, 2 ** 18 + 5, np.float32))      # bf16 bit patterns
    pb, gb, mb, vb = (dev(x, bf16=True) for x in (p, g, m, v))
    p32, g32, m32, v32 = (oracle.bf16_widen(x) for x in (p, g, m, v))
    api.adam_step(pb, gb, mb, vb, lr=0.01)
    exp_p, exp_m, exp_v = oracle.adam_step(p32, g32, m32, v32, lr=0.01, bf16=True)
    assert np.array_equal(oracle.bf16_widen(host(mb)), exp_m)
    assert np.array_equal(oracle.bf16_widen(host(vb)), exp_v)
    assert np.array_equal(oracle.bf16_widen(host(pb)), exp_p, equal_nan=True)
    api.sgd_step(pb, gb, lr=0.1)
    assert np.array_equal(oracle.bf16_widen(host(pb)), oracle.sgd_step(exp_p, g32, lr=0.1, bf16=True), equal_nan=True)
    lib = _lib.lib()
    xi = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert lib.ntb200_sgd_step(_lib.I32, xi.data_ptr(), xi.data_ptr(), 8, 0.1, None) == _lib.ERR_UNSUPPORTED
    assert lib.ntb200_adam_step(_lib.F32, None, xi.data_ptr(), xi.data_ptr(), xi.data_ptr(), 8, 0.1, 0.9, 0.999, 1e-8, 0,
                                None) == _lib.ERR_INVALID_ARG
    with pytest.raises(ValueError):
        api.sgd_step(torch.zeros((4, 4), device="cuda").t(), torch.zeros((4, 4), device="cuda"))
