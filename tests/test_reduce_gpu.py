"""Parity of tb200_reduce (through the C ABI) with the CPU oracle.

Mirrors the reference's reduce tests: the known answer with and without an initial value
(testing/reduce.cu:26-38), all sizes on integral types with an initial value
(testing/reduce.cu:79-96); bit-exact for integers of every width (sums wrap), floating point
within 1e-5 of the sum of absolute values (association order differs), plus pointers that are
not 16-byte aligned and the committed reference vectors.
"""
from pathlib import Path

import numpy as np
import pytest

import oracle
import thrust_b200 as tb
from util import to_device

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 2, 31, 33, 1000, 8191, 8192, 8193, 100003, (1 << 21) + 13, (1 << 25) + 7]
INT_TYPES = [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64]
FLT_TYPES = [np.float32, np.float64]


def _data(rng, n, dtype):
    if np.dtype(dtype).kind == "f":
        return rng.uniform(-1, 1, size=n).astype(dtype)
    ii = np.iinfo(dtype)
    return rng.integers(ii.min, ii.max, size=n, dtype=dtype, endpoint=True)  # wraps, like the reference


def test_reduce_known_answer(cuda_device):
    for dtype in (np.int8, np.int32, np.int64, np.float32, np.float64):
        d = to_device(np.array([1, -2, 3], dtype=dtype))
        assert tb.reduce(d) == 2
        assert tb.reduce(d, 10) == 12


@pytest.mark.parametrize("dtype", INT_TYPES)
def test_reduce_integers_bit_exact(cuda_device, dtype):
    chk = oracle.port()
    for n in SIZES:
        rng = np.random.default_rng(11 + n)
        a = _data(rng, n, dtype)
        for off in (0, 1):  # off = 1: the input starts one element past a 16-byte boundary
            d = to_device(a, offset_elems=off)
            for init in (None, 13):
                want = chk.reduce(a, init)
                got = tb.reduce(d, init)
                assert np.array([got], dtype=dtype).tobytes() == np.array([want]).tobytes(), (n, off, init)


@pytest.mark.parametrize("dtype", FLT_TYPES)
def test_reduce_floats_within_tolerance(cuda_device, dtype):
    chk = oracle.port()
    for n in SIZES:
        rng = np.random.default_rng(110 + n)
        a = _data(rng, n, dtype)
        d = to_device(a)
        tol = 1e-5 * float(np.abs(a.astype(np.float64)).sum()) + 1e-30
        exact = float(a.astype(np.float64).sum())
        for init in (None, 0.5):
            want = float(chk.reduce(a, init))
            got = float(tb.reduce(d, init))
            assert abs(got - want) <= tol, (n, init, got, want)
            assert abs(got - (exact + (init or 0.0))) <= tol, (n, init)
        if n:  # reproducible from run to run
            assert tb.reduce(d) == tb.reduce(d)


@pytest.mark.parametrize("t", ["int8", "uint8", "int16", "uint16", "int32", "uint32", "int64", "uint64"])
def test_reduce_matches_committed_reference_vectors(cuda_device, t):
    v = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
    a = v[f"reduce/{t}/in"]
    d = to_device(a)
    assert np.array([tb.reduce(d)], dtype=a.dtype).tobytes() == v[f"reduce/{t}/sum"].tobytes()
    assert np.array([tb.reduce(d, 13)], dtype=a.dtype).tobytes() == v[f"reduce/{t}/sum_init13"].tobytes()
