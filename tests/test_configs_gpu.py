"""The BASELINE configurations at FULL size on the GPU: complete oracle comparison where the oracle finishes
in seconds, and size-independent properties (checksum of checksums, linearity, batch independence) elsewhere.
Inputs follow the measurement plan: seeded synthetic tensors with the stated shapes and distributions."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host, integers, normal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from neurotensor_b200 import api as a
    return a


def test_config2_batched_f16_transposed_view(api, oracle):
    """fp16 [64,2048,2048] x transposed view of [64,2048,2048], fp32 accumulate."""
    from neurotensor_b200 import _lib
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.randn((64, 2048, 2048), generator=gen, device="cuda") * 0.1).half()
    bs = (torch.randn((64, 2048, 2048), generator=gen, device="cuda") * 0.1).half()
    b = bs.transpose(-1, -2)
    c = api.matmult(a, b)
    assert _lib.last_route() == "umma_f16" and tuple(c.shape) == (64, 2048, 2048)
    # full oracle comparison on three batch items
    for i in (0, 31, 63):
        exp = oracle.matmult(host(a[i]), host(bs[i]), False, True)
        assert oracle.rel_fro(host(c[i]), exp) <= 2e-3
    # checksum of checksums on every item, in float64 on the host: (A.B).1 == A.(B.1)
    ones = torch.ones((2048, 1), dtype=torch.float64, device="cuda")
    lhs = (c.double() @ ones).squeeze(-1)
    rhs = (a.double() @ (b.double() @ ones)).squeeze(-1)
    err = (lhs - rhs).norm() / rhs.norm()
    assert err.item() <= 2e-3
    # batch independence: item 5 computed alone equals item 5 of the batch, bit for bit
    alone = api.matmult(a[5], b[5])
    assert torch.equal(alone, c[5])


def test_config3_int8_full_size_bit_exact(api, oracle):
    rng = np.random.default_rng(5)
    a, b = integers(rng, (4096, 8192), np.int8, -8, 7), integers(rng, (8192, 4096), np.int8, -8, 7)
    got = host(api.matmult(dev(a), dev(b)))
    from neurotensor_b200 import _lib
    assert _lib.last_route() == "umma_i8"
    assert got.dtype == np.int8
    assert np.array_equal(got, oracle.matmult(a, b))


def test_config3_int32_full_size_bit_exact(api, oracle):
    rng = np.random.default_rng(7)
    a, b = integers(rng, (2048, 2048), np.int32, -1000, 1000), integers(rng, (2048, 2048), np.int32, -1000, 1000)
    assert np.array_equal(host(api.matmult(dev(a), dev(b))), oracle.matmult(a, b))


def test_config4_mlp_gemms_full_size(api, oracle):
    """bf16 8192 x (4096 -> 16384): row slabs against the oracle, and linearity on the full problem."""
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((8192, 4096), generator=gen, device="cuda").bfloat16()
    w1 = (torch.randn((4096, 16384), generator=gen, device="cuda") * 4096 ** -0.5).bfloat16()
    h = api.matmult(x, w1)
    rows = slice(4000, 4064)
    exp = oracle.matmult(host(x[rows]), host(w1), bf16=True)
    assert oracle.rel_fro(oracle.bf16_widen(host(h[rows])), oracle.bf16_widen(exp)) <= 2e-3
    # dW = x^T . g without materialising the transpose (flag only)
    g = torch.randn((8192, 512), generator=gen, device="cuda").bfloat16()
    dw = api.matmult(x, g, True, False)
    cols = slice(100, 164)
    exp_dw = oracle.matmult(host(x[:, cols].contiguous()), host(g), True, False, bf16=True)
    assert oracle.rel_fro(oracle.bf16_widen(host(dw[cols])), oracle.bf16_widen(exp_dw)) <= 2e-3
    # linearity in the first operand: (2x).W == 2 (x.W) exactly in binary floating point
    h2 = api.matmult(x * 2, w1)
    assert torch.equal(h2, h * 2)


def test_config5_conv2d_full_size(api, oracle):
    gen = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn((32, 256, 56, 56), generator=gen, device="cuda").half()
    w = (torch.randn((256, 256, 3, 3), generator=gen, device="cuda") * (256 * 9) ** -0.5).half()
    out = api.conv2d(x, w, stride=1, padding=1)
    assert tuple(out.shape) == (32, 256, 56, 56)
    exp = oracle.conv2d(host(x[7:8]), host(w), stride=1, padding=1)
    assert oracle.rel_fro(host(out[7:8]), exp) <= 2e-3
    # images are independent: the first image alone gives the same bits
    assert torch.equal(api.conv2d(x[:1], w, stride=1, padding=1), out[:1])


@pytest.mark.parametrize("n", [512, 2048])
def test_config5_f32_sweep_points(api, oracle, n):
    from neurotensor_b200 import _lib
    rng = np.random.default_rng(16 + n)
    a, b = normal(rng, (n, n), np.float32), normal(rng, (n, n), np.float32)
    exp = oracle.matmult(a, b)
    assert oracle.rel_fro(host(api.matmult(dev(a), dev(b))), exp) <= 1e-5          # tensor cores, 3 x TF32
    assert _lib.last_route() == "umma_3xtf32"
    assert np.array_equal(host(api.matmult(dev(a), dev(b), route=_lib.ROUTE_SIMT)), exp)   # CUDA cores: bit-exact
