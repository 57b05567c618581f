"""Parity of tb200_reduce_by_key (through the C ABI) with the CPU oracle.

Mirrors the reference's tests: the 9-element known answer (testing/reduce_by_key.cu:47-112)
and TestReduceByKey (testing/reduce_by_key.cu:115-156: keys from random bools, so run lengths
are geometric with mean 2, unsigned int values, every size; counts, keys and sums compared
bit-exactly). Floating-point sums are compared within 1e-5 of the run's sum of absolute values.
"""
import numpy as np
import pytest

import oracle
import thrust_b200 as tb
from util import to_device, to_host

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 2, 3, 31, 32, 33, 1000, 2047, 2048, 2049, 4095, 4096, 4097, 8193, 10007, 65537, (1 << 20) + 13]


def _grouped_keys(rng, n, p_new, dtype):
    """Already-grouped keys: a new run starts with probability p_new."""
    heads = rng.random(n) < p_new
    ids = np.cumsum(heads)
    if np.dtype(dtype).itemsize == 1:
        ids = ids % 2  # narrow keys: alternate so neighbouring runs still differ
    return ids.astype(dtype)


def _run(keys, vals):
    dk, dv = to_device(keys), to_device(vals)
    ko, vo, r = tb.reduce_by_key(dk, dv)
    assert to_host(dk, keys.dtype).tobytes() == keys.tobytes()
    assert to_host(dv, vals.dtype).tobytes() == vals.tobytes()
    return to_host(ko, keys.dtype)[:r], to_host(vo, vals.dtype)[:r]


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("kdtype", [np.int32, np.uint64, np.uint8, np.int16])
def test_rbk_integers_bit_exact(cuda_device, n, kdtype):
    rng = np.random.default_rng(11 + n)
    chk = oracle.port()
    for p_new, vdtype in [(0.5, np.uint32), (1 / 16, np.int64), (1.0, np.int32), (0.0005, np.uint64)]:
        keys = _grouped_keys(rng, n, p_new, kdtype)
        vals = rng.integers(0, 1 << 31, size=n).astype(vdtype)
        wk, wv = chk.reduce_by_key(keys, vals)
        gk, gv = _run(keys, vals)
        assert gk.shape == wk.shape, (p_new, vdtype)
        assert gk.tobytes() == wk.tobytes()
        assert gv.tobytes() == wv.tobytes()


@pytest.mark.parametrize("kdtype,vdtype", [(np.int32, np.int32), (np.uint64, np.int64), (np.int32, np.uint64)])
def test_rbk_integers_bit_exact_many_tiles_per_cta(cuda_device, kdtype, vdtype):
    # enough tiles that every persistent CTA refills its ring several times (tickets, slot reuse)
    n = (1 << 23) + 13
    rng = np.random.default_rng(n)
    chk = oracle.port()
    for p_new in (1 / 16, 0.9, 0.00001):
        keys = _grouped_keys(rng, n, p_new, kdtype)
        vals = rng.integers(0, 1 << 31, size=n).astype(vdtype)
        wk, wv = chk.reduce_by_key(keys, vals)
        gk, gv = _run(keys, vals)
        assert gk.shape == wk.shape, p_new
        assert gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes(), p_new


@pytest.mark.parametrize("n", [0, 1, 4097, 100003, (1 << 22) + 5])
@pytest.mark.parametrize("vdtype", [np.float32, np.float64])
def test_rbk_float_values_within_tolerance(cuda_device, n, vdtype):
    rng = np.random.default_rng(110 + n)
    chk = oracle.port()
    keys = _grouped_keys(rng, n, 1 / 16, np.int32)
    vals = rng.uniform(-50, 50, size=n).astype(vdtype)
    wk, wv = chk.reduce_by_key(keys, vals)
    gk, gv = _run(keys, vals)
    assert gk.tobytes() == wk.tobytes()
    if n:
        # per-run tolerance: 1e-5 x sum |v| of that run
        heads = np.flatnonzero(np.r_[True, keys[1:] != keys[:-1]])
        abs_sums = np.add.reduceat(np.abs(vals.astype(np.float64)), heads)
        assert np.all(np.abs(gv.astype(np.float64) - wv.astype(np.float64)) <= 1e-5 * abs_sums + 1e-30)


def test_rbk_one_long_run_spans_many_tiles(cuda_device):
    n = 300001
    keys = np.full(n, 7, dtype=np.int32)
    vals = np.arange(n, dtype=np.int64)
    gk, gv = _run(keys, vals)
    assert gk.tolist() == [7] and gv.tolist() == [n * (n - 1) // 2]


def test_rbk_float_keys_ieee_equality(cuda_device):
    keys = np.array([0.0, -0.0, 1.5, 1.5, np.nan, np.nan, 2.0], dtype=np.float32)
    vals = np.arange(1, 8, dtype=np.int32)
    wk, wv = oracle.port().reduce_by_key(keys, vals)
    gk, gv = _run(keys, vals)
    assert gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes()
    assert gv.tolist() == [3, 7, 5, 6, 7]


def test_rbk_known_answer(cuda_device):
    # testing/reduce_by_key.cu:15-42: keys 11 11 21 20 21 21 21 37 37, values 0..8
    keys = np.array([11, 11, 21, 20, 21, 21, 21, 37, 37], dtype=np.int32)
    vals = np.arange(9, dtype=np.int32)
    gk, gv = _run(keys, vals)
    assert gk.tolist() == [11, 21, 20, 21, 37]
    assert gv.tolist() == [1, 2, 3, 15, 15]


def test_rbk_unaligned_pointers(cuda_device):
    rng = np.random.default_rng(3)
    n = 70001
    keys = _grouped_keys(rng, n, 0.1, np.int32)
    vals = rng.integers(0, 1000, size=n).astype(np.int32)
    dk, dv = to_device(keys, offset_elems=1), to_device(vals, offset_elems=3)
    ko, vo, r = tb.reduce_by_key(dk, dv)
    wk, wv = oracle.port().reduce_by_key(keys, vals)
    assert r == wk.size
    assert to_host(ko, np.int32)[:r].tobytes() == wk.tobytes()
    assert to_host(vo, np.int32)[:r].tobytes() == wv.tobytes()
