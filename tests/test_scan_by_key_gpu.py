"""Parity of tb200_scan_by_key (through the C ABI) with the CPU oracle.

Mirrors the reference's scan_by_key tests: the known answers with and without an initial value
(testing/scan_by_key.inclusive.cu:12-60, testing/scan_by_key.exclusive.cu), all sizes with
random run lengths, in place on the values (testing/scan_by_key.inclusive.cu:288-336);
bit-exact for integer values, floating point within 1e-5 of the sum of absolute values.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
import thrust_b200 as tb
from util import to_device, to_host

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 2, 33, 1000, 8191, 8192, 8193, 100003, (1 << 21) + 13]


def _keys(rng, n, dtype, p):
    return np.cumsum(rng.random(n) < p).astype(dtype)


def test_scan_by_key_known_answers(cuda_device):
    k = to_device(np.array([0, 1, 1, 1, 2, 3, 3], dtype=np.int32))
    v = to_device(np.array([1, 2, 3, 4, 5, 6, 7], dtype=np.int32))
    assert tb.inclusive_scan_by_key(k, v).cpu().tolist() == [1, 2, 5, 9, 5, 6, 13]
    assert tb.exclusive_scan_by_key(k, v).cpu().tolist() == [0, 0, 2, 5, 0, 0, 6]
    assert tb.exclusive_scan_by_key(k, v, init=10).cpu().tolist() == [10, 10, 12, 15, 10, 10, 16]


@pytest.mark.parametrize("kdtype", [np.uint8, np.int16, np.int32, np.uint64, np.float32])
@pytest.mark.parametrize("vdtype", [np.int32, np.uint64])
def test_scan_by_key_integers_bit_exact(cuda_device, kdtype, vdtype):
    chk = oracle.port()
    for n in SIZES:
        rng = np.random.default_rng(300 + n)
        for p in (1 / 16, 0.5, 0.0005):
            k = _keys(rng, n, kdtype, p)
            ii = np.iinfo(vdtype)
            v = rng.integers(ii.min, ii.max, size=n, dtype=vdtype, endpoint=True)  # sums wrap
            for off in (0, 1):  # off = 1: pointers one element past a 16-byte boundary
                dk, dv = to_device(k, offset_elems=off), to_device(v, offset_elems=off)
                for ex, init in [(False, None), (True, None), (True, 11)]:
                    want = chk.scan_by_key(k, v, ex, init)
                    got = tb.exclusive_scan_by_key(dk, dv, init=init) if ex else tb.inclusive_scan_by_key(dk, dv)
                    assert to_host(got, vdtype).tobytes() == want.tobytes(), (n, p, off, ex, init)
                    assert to_host(dv, vdtype).tobytes() == v.tobytes(), "values modified"
            # in place on the values
            dk, dv = to_device(k), to_device(v)
            tb.inclusive_scan_by_key(dk, dv, out=dv)
            assert to_host(dv, vdtype).tobytes() == chk.scan_by_key(k, v).tobytes(), (n, p)


@pytest.mark.parametrize("kdtype,vdtype", [(np.int32, np.int32), (np.uint64, np.int64), (np.uint8, np.uint64)])
def test_scan_by_key_integers_bit_exact_many_tiles_per_cta(cuda_device, kdtype, vdtype):
    # enough tiles that every persistent CTA refills its ring several times (tickets, slot reuse)
    n = (1 << 23) + 13
    rng = np.random.default_rng(n)
    chk = oracle.port()
    for p in (1 / 16, 0.9, 0.00001):
        k = _keys(rng, n, kdtype, p)
        ii = np.iinfo(vdtype)
        v = rng.integers(ii.min, ii.max, size=n, dtype=vdtype, endpoint=True)
        dk, dv = to_device(k), to_device(v)
        assert to_host(tb.inclusive_scan_by_key(dk, dv), vdtype).tobytes() == chk.scan_by_key(k, v).tobytes(), p
        assert to_host(tb.exclusive_scan_by_key(dk, dv, init=7), vdtype).tobytes() == \
            chk.scan_by_key(k, v, True, 7).tobytes(), p
        tb.inclusive_scan_by_key(dk, dv, out=dv)
        assert to_host(dv, vdtype).tobytes() == chk.scan_by_key(k, v).tobytes(), p


@pytest.mark.parametrize("vdtype", [np.float32, np.float64])
def test_scan_by_key_floats_within_tolerance(cuda_device, vdtype):
    chk = oracle.port()
    for n in [0, 1, 5, 8193, 100003, (1 << 22) + 5]:
        rng = np.random.default_rng(400 + n)
        for p in (1 / 16, 0.0005):
            k = _keys(rng, n, np.int32, p)
            v = rng.uniform(-50, 50, size=n).astype(vdtype)
            dk, dv = to_device(k), to_device(v)
            tol = 1e-5 * float(np.abs(v.astype(np.float64)).sum()) + 1e-30
            for ex, init in [(False, None), (True, None), (True, 0.5)]:
                want = chk.scan_by_key(k, v, ex, init).astype(np.float64)
                got = tb.exclusive_scan_by_key(dk, dv, init=init) if ex else tb.inclusive_scan_by_key(dk, dv)
                got = to_host(got, vdtype).astype(np.float64)
                assert got.shape == want.shape
                if n:
                    assert float(np.max(np.abs(got - want))) <= tol, (n, p, ex, init)


@pytest.mark.parametrize("t", ["int32", "uint32", "int64", "uint64"])
def test_scan_by_key_matches_committed_reference_vectors(cuda_device, t):
    v = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
    keys, vals = v[f"sbk/{t}/keys"], v[f"sbk/{t}/vals"]
    dk, dv = to_device(keys), to_device(vals)
    assert to_host(tb.inclusive_scan_by_key(dk, dv), vals.dtype).tobytes() == v[f"sbk/{t}/inclusive"].tobytes()
    assert to_host(tb.exclusive_scan_by_key(dk, dv), vals.dtype).tobytes() == v[f"sbk/{t}/exclusive"].tobytes()
    assert to_host(tb.exclusive_scan_by_key(dk, dv, init=11), vals.dtype).tobytes() == \
        v[f"sbk/{t}/exclusive_init11"].tobytes()
