"""The oracle (oracle/oracle.cpp, a restatement) against the REFERENCE's own matmult kernel, compiled from the
reference's sources by oracle/build_ref.py (nt_matmult.hpp + nt_matmult_simde.hpp + the per-dtype SIMD traits, with
stand-ins only for the un-vendored simde / oneTBB / half headers).  Bit for bit, every dtype the kernel vectorises,
all four transpose combinations, ragged shapes that leave partial tiles in every direction, and the raw C += contract.
This is what pins the Float16 (fp16 rounding of the running sum at every 16-k boundary) and the integer (wrap in the
operands' own width) rows, for which the reference's tests hold no vector.

Where neither the reference tree nor a prebuilt library is present the module is skipped."""
import ctypes

import numpy as np
import pytest

from conftest import ROOT  # noqa: F401  (puts the repository root on sys.path)
from oracle import build_ref

LIB = build_ref.build()
if LIB is None:
    pytest.skip("no reference tree and no prebuilt oracle/_ref/libntref.so", allow_module_level=True)
REF = ctypes.CDLL(LIB)
REF.ntref_matmult.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 4 + [ctypes.c_int] * 2
CODES = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.int8): 3, np.dtype(np.int16): 4, np.dtype(np.int32): 5,
         np.dtype(np.int64): 6, np.dtype(np.float64): 7, np.dtype(np.uint8): 8}


def reference_matmult_into(a, b, c, ta, tb):
    """nt_matmult<T>(A, B, C, a_rows, a_cols, b_rows, b_cols, ta, tb): C += op(A).op(B); dims are the logical ones
    after the transposes (nt/functional/cpu/matmult/nt_matmult.h:6-7)."""
    m, k = (a.shape[1], a.shape[0]) if ta else a.shape
    k2, n = (b.shape[1], b.shape[0]) if tb else b.shape
    assert k == k2 and c.shape == (m, n)
    rc = REF.ntref_matmult(CODES[a.dtype], a.ctypes.data, b.ctypes.data, c.ctypes.data, m, k, k2, n, int(ta), int(tb))
    assert rc == 0
    return c


def make(rng, shape, dtype):
    if np.issubdtype(dtype, np.floating):
        return (rng.standard_normal(shape) * 0.5).astype(dtype)
    info = np.iinfo(dtype)
    return rng.integers(info.min, info.max, size=shape, endpoint=True).astype(dtype)     # full range: wraps everywhere


SHAPES = [(1, 1, 1), (7, 5, 3), (16, 16, 16), (17, 33, 19), (64, 100, 48), (130, 47, 129), (70, 2304, 40), (33, 257, 65)]


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.int8, np.uint8, np.int16, np.int32, np.int64, np.float64])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_oracle_equals_the_reference_kernel_bit_for_bit(oracle, dtype, ta, tb):
    rng = np.random.default_rng(11)
    for m, k, n in SHAPES:
        a = make(rng, (k, m) if ta else (m, k), dtype)
        b = make(rng, (n, k) if tb else (k, n), dtype)
        c0 = make(rng, (m, n), dtype)
        want = reference_matmult_into(a, b, c0.copy(), ta, tb)
        got = oracle.matmult_into(a, b, c0.copy(), ta, tb)
        assert got.tobytes() == want.tobytes(), (np.dtype(dtype).name, m, k, n, ta, tb)
        # and from a zero-filled C, which is how functional::matmult calls it (matmult_cpu.cpp:110)
        want0 = reference_matmult_into(a, b, np.zeros((m, n), dtype), ta, tb)
        assert oracle.matmult(a, b, ta, tb).tobytes() == want0.tobytes()


def test_complex_types_on_the_reference_kernel(oracle):
    """Complex64 and Complex32: the reference multiplies real parts with real parts and imaginary parts with imaginary
    parts (its traits are the lane operations on interleaved data), Complex32 rounding to Float16 every 8 k-steps; the
    oracle reproduces both bit for bit.  Complex128: the reference's kernel returns with C untouched -- the switch that
    loads and stores the C tile has cases for tile sizes 64, 32, 16 and 8 only (nt_matmult_macros.h:413-438) and this
    type's tile is 4 wide -- so functional::matmult of two Complex128 tensors is all zeros there.  That is recorded
    here as a fact about the reference; the library computes the lane-wise product its traits define, like Complex64."""
    rng = np.random.default_rng(13)
    for m, k, n in SHAPES[:6]:
        for ta in (False, True):
            for tb in (False, True):
                sa, sb = ((k, m) if ta else (m, k)), ((n, k) if tb else (k, n))
                a = (rng.standard_normal(sa) + 1j * rng.standard_normal(sa)).astype(np.complex64)
                b = (rng.standard_normal(sb) + 1j * rng.standard_normal(sb)).astype(np.complex64)
                c = np.zeros((m, n), np.complex64)
                assert REF.ntref_matmult(11, a.ctypes.data, b.ctypes.data, c.ctypes.data, m, k, k, n, int(ta), int(tb)) == 0
                assert oracle.matmult(a, b, ta, tb).tobytes() == c.tobytes()
                ah, bh = rng.standard_normal(sa + (2,)).astype(np.float16), rng.standard_normal(sb + (2,)).astype(np.float16)
                ch = np.zeros((m, n, 2), np.float16)
                assert REF.ntref_matmult(13, ah.ctypes.data, bh.ctypes.data, ch.ctypes.data, m, k, k, n, int(ta), int(tb)) == 0
                assert oracle.matmult_complex32(ah, bh, ta, tb).tobytes() == ch.tobytes()
    a = (rng.standard_normal((8, 8)) + 1j * rng.standard_normal((8, 8))).astype(np.complex128)
    c0 = np.full((8, 8), 1 + 2j, np.complex128)
    c = c0.copy()
    assert REF.ntref_matmult(12, a.ctypes.data, a.ctypes.data, c.ctypes.data, 8, 8, 8, 8, 0, 0) == 0
    assert np.array_equal(c, c0)            # untouched: no tile-size-4 case in the reference's load / store switch


def test_float16_rounds_the_running_sum_every_16_k(oracle):
    """The property the Float16 parity bars rest on, seen on the reference kernel itself: its result differs from an
    fp32-accumulate-and-round-once product, by the amounts the oracle predicts."""
    rng = np.random.default_rng(3)
    for k, lo, hi in ((2048, 1.4e-3, 2.0e-3), (8192, 2.8e-3, 3.8e-3)):
        a = (rng.standard_normal((64, k)) * 0.1).astype(np.float16)
        b = (rng.standard_normal((k, 64)) * 0.1).astype(np.float16)
        ref = reference_matmult_into(a, b, np.zeros((64, 64), np.float16), False, False)
        once = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32).astype(np.float16)
        d = oracle.rel_fro(ref, once)
        assert lo < d < hi, (k, d)
        assert oracle.matmult(a, b).tobytes() == ref.tobytes()
