"""Parity of tb200_scan (through the C ABI) with the CPU oracle.

Mirrors the reference's scan tests: known answers and in-place forms
(testing/scan.cu:26-107), all sizes on integral types with inclusive / exclusive /
init / in-place (testing/scan.cu:379-415), bit-exact for integers; floating point
within 1e-5 of the sum of absolute values (association order differs).
"""
import numpy as np
import pytest
import torch

import oracle
import thrust_b200 as tb
from util import to_device, to_host

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 2, 31, 32, 33, 1000, 2047, 2048, 2049, 4095, 4096, 4097, 10007, 65536, (1 << 20) + 13]
INT_TYPES = [np.int32, np.uint32, np.int64, np.uint64]
FLT_TYPES = [np.float32, np.float64]


def _data(rng, n, dtype):
    if np.dtype(dtype).kind == "f":
        return rng.uniform(-1, 1, size=n).astype(dtype)
    ii = np.iinfo(dtype)
    return rng.integers(ii.min, ii.max, size=n, dtype=dtype, endpoint=True)  # wraps, like the reference


@pytest.mark.parametrize("dtype", INT_TYPES)
@pytest.mark.parametrize("n", SIZES)
def test_scan_integers_bit_exact(cuda_device, dtype, n):
    rng = np.random.default_rng(7 + n)
    a = _data(rng, n, dtype)
    chk = oracle.port()
    d = to_device(a)
    for exclusive, init in [(False, None), (True, None), (True, 11)]:
        want = chk.scan(a, exclusive, init)
        got = tb.exclusive_scan(d, init=init) if exclusive else tb.inclusive_scan(d)
        assert to_host(got, dtype).tobytes() == want.tobytes(), (exclusive, init)
        assert to_host(d, dtype).tobytes() == a.tobytes(), "input modified"
    # exactly in place
    e = d.clone()
    tb.inclusive_scan(e, out=e)
    assert to_host(e, dtype).tobytes() == chk.scan(a).tobytes()
    e = d.clone()
    tb.exclusive_scan(e, out=e, init=3)
    assert to_host(e, dtype).tobytes() == chk.scan(a, True, 3).tobytes()


@pytest.mark.parametrize("dtype", [np.int32, np.uint64])
@pytest.mark.parametrize("n", [(1 << 23) + 13, (1 << 24) + 7])
def test_scan_integers_bit_exact_many_tiles_per_cta(cuda_device, dtype, n):
    # enough tiles that every persistent CTA refills its ring several times (tickets, slot reuse)
    rng = np.random.default_rng(n)
    a = _data(rng, n, dtype)
    chk = oracle.port()
    d = to_device(a)
    assert to_host(tb.inclusive_scan(d), dtype).tobytes() == chk.scan(a).tobytes()
    assert to_host(tb.exclusive_scan(d, init=5), dtype).tobytes() == chk.scan(a, True, 5).tobytes()
    tb.inclusive_scan(d, out=d)
    assert to_host(d, dtype).tobytes() == chk.scan(a).tobytes()


@pytest.mark.parametrize("dtype", FLT_TYPES)
@pytest.mark.parametrize("n", [0, 1, 5, 4097, 100003, (1 << 22) + 5])
def test_scan_floats_within_tolerance(cuda_device, dtype, n):
    rng = np.random.default_rng(70 + n)
    a = _data(rng, n, dtype)
    d = to_device(a)
    chk = oracle.port()
    tol = 1e-5 * float(np.abs(a.astype(np.float64)).sum()) + 1e-30
    for exclusive, init in [(False, None), (True, None), (True, 0.5)]:
        want = chk.scan(a, exclusive, init).astype(np.float64)
        got = tb.exclusive_scan(d, init=init) if exclusive else tb.inclusive_scan(d)
        got = to_host(got, dtype).astype(np.float64)
        assert got.shape == want.shape
        if n:
            assert np.max(np.abs(got - want)) <= tol


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32])
def test_scan_unaligned_pointers(cuda_device, dtype):
    rng = np.random.default_rng(5)
    n = 50001
    a = rng.integers(-1000, 1000, size=n).astype(dtype)
    d = to_device(a, offset_elems=1)
    assert d.data_ptr() % 16 != 0
    out = to_device(np.zeros(n, dtype=dtype), offset_elems=3 if np.dtype(dtype).itemsize == 4 else 1)
    tb.inclusive_scan(d, out=out)
    assert to_host(out, dtype).tobytes() == oracle.port().scan(a).tobytes()


def test_scan_known_answers(cuda_device):
    # the five-element vector of the reference's TestScanSimple (testing/scan.cu:44-104)
    a = np.array([1, 3, -2, 4, -5], dtype=np.int32)
    d = to_device(a)
    assert to_host(tb.inclusive_scan(d), np.int32).tolist() == [1, 4, 2, 6, 1]
    assert to_host(tb.exclusive_scan(d), np.int32).tolist() == [0, 1, 4, 2, 6]
    assert to_host(tb.exclusive_scan(d, init=3), np.int32).tolist() == [3, 4, 7, 5, 9]


def test_scan_rejects_bad_arguments(cuda_device):
    with pytest.raises(TypeError):
        tb.inclusive_scan(torch.zeros(8, dtype=torch.int16, device="cuda"))
    with pytest.raises(ValueError):
        tb.inclusive_scan(torch.zeros(8, dtype=torch.int32))


@pytest.mark.parametrize("dtype", [np.int32, np.uint64])
@pytest.mark.parametrize("n", [1, 33, 4097, (1 << 20) + 13, (1 << 23) + 5])
def test_seeded_inclusive_scan_bit_exact(cuda_device, dtype, n):
    # out[i] = seed + in[0] + ... + in[i]: what a shard of a distributed scan runs
    rng = np.random.default_rng(70 + n)
    a = _data(rng, n, dtype)
    with np.errstate(over="ignore"):
        want = (oracle.port().scan(a, True, 12345) + a).astype(dtype)
    got = tb.inclusive_scan(to_device(a), init=12345)
    assert to_host(got, dtype).tobytes() == want.tobytes()


def test_sharded_scan_and_reduce_by_key_on_one_rank_match_the_oracle(cuda_device):
    from thrust_b200.sharded_scan import ShardedScan
    rng = np.random.default_rng(5)
    n = (1 << 20) + 77
    vals = rng.integers(-1000, 1000, size=n, dtype=np.int64)
    keys = np.cumsum(rng.random(n) < 1 / 16).astype(np.int32)
    chk = oracle.port()
    sh = ShardedScan(1, 0)
    dv, dk = to_device(vals), to_device(keys)
    assert to_host(sh.inclusive_scan(dv), np.int64).tobytes() == chk.scan(vals).tobytes()
    assert to_host(sh.exclusive_scan(dv, init=3), np.int64).tobytes() == chk.scan(vals, True, 3).tobytes()
    ko, vo, m = sh.reduce_by_key(dk, dv)
    wk, wv = chk.reduce_by_key(keys, vals)
    assert m == wk.size and to_host(ko[:m], np.int32).tobytes() == wk.tobytes()
    assert to_host(vo[:m], np.int64).tobytes() == wv.tobytes()
