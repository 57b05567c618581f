"""Parity of tb200_unique_by_key and tb200_copy_flagged (through the C ABI) with the CPU oracle.

Mirrors the reference's tests: the 9-element known answer of testing/unique_by_key.cu:127-207
(in place and copying), TestUniqueByKey / TestUniqueCopyByKey (testing/unique_by_key.cu:250-330:
random keys with short runs, every size, outputs compared element for element) and the stencil
form of copy_if (testing/copy.cu:400-430). Everything is compared bit for bit: keys are only
compared and values only moved.
"""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
import thrust_b200 as tb
from util import to_device, to_host

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
# 5120 / 2560 / 1280 are tile sizes of the streaming kernel (4-, 8-, 16-byte elements)
SIZES = [0, 1, 2, 33, 1279, 1280, 1281, 2559, 2560, 2561, 5119, 5120, 5121, 10007, 65537, 40 * 5120 + 17,
         (1 << 20) + 13]
KEY_TYPES = [np.int8, np.uint16, np.int32, np.uint64, np.float32, np.float64]


def _runs(rng, n, p_new, dtype):
    ids = np.cumsum(rng.random(n) < p_new)
    if np.dtype(dtype).itemsize == 1:
        ids = ids % 2
    return ids.astype(dtype)


def _unique(keys, vals, inplace, offset=0):
    dk = to_device(keys, offset_elems=offset)
    dv = None if vals is None else to_device(vals, offset_elems=offset)
    ko, vo, r = tb.unique_by_key(dk, dv, inplace=inplace)
    if not inplace:
        assert to_host(dk, keys.dtype).tobytes() == keys.tobytes()
    return to_host(ko, keys.dtype)[:r], (None if vals is None else to_host(vo, vals.dtype)[:r])


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("kdtype", KEY_TYPES)
def test_unique_by_key_bit_exact(cuda_device, n, kdtype):
    rng = np.random.default_rng(23 + n)
    chk = oracle.port()
    for p_new, vdtype in [(0.5, np.uint32), (1 / 16, np.uint64), (1.0, np.uint8), (0.0005, np.uint16), (0.3, None)]:
        keys = _runs(rng, n, p_new, kdtype)
        vals = None if vdtype is None else rng.integers(0, 250, size=n).astype(vdtype)
        wk, wv = chk.unique_by_key(keys, vals)
        for inplace in (False, True):
            gk, gv = _unique(keys, vals, inplace)
            assert gk.shape == wk.shape, (p_new, vdtype, inplace)
            assert gk.tobytes() == wk.tobytes(), (p_new, vdtype, inplace)
            assert vals is None or gv.tobytes() == wv.tobytes(), (p_new, vdtype, inplace)


@pytest.mark.parametrize("kdtype,vdtype", [(np.int32, np.uint32), (np.uint64, np.uint64), (np.int32, None)])
def test_select_bit_exact_many_tiles_per_cta(cuda_device, kdtype, vdtype):
    # enough tiles that every persistent CTA refills its ring several times (tickets, slot reuse)
    n = (1 << 23) + 13
    rng = np.random.default_rng(n)
    chk = oracle.port()
    for p in (1 / 16, 0.9, 0.00001):
        keys = _runs(rng, n, p, kdtype)
        vals = None if vdtype is None else rng.integers(0, 1 << 31, size=n).astype(vdtype)
        wk, wv = chk.unique_by_key(keys, vals)
        for inplace in (False, True):
            gk, gv = _unique(keys, vals, inplace)
            assert gk.tobytes() == wk.tobytes(), (p, inplace)
            assert vals is None or gv.tobytes() == wv.tobytes(), (p, inplace)
        if vals is not None:
            flags = (rng.random(n) < p).astype(np.uint8)
            out, r = tb.copy_flagged(to_device(vals), to_device(flags))
            assert to_host(out, vals.dtype)[:r].tobytes() == chk.copy_flagged(vals, flags).tobytes(), p


def test_unique_by_key_16_byte_values(cuda_device):
    rng = np.random.default_rng(16)
    n = 100003
    keys = _runs(rng, n, 0.25, np.int32)
    vals = rng.integers(0, 1 << 63, size=(n, 2), dtype=np.uint64)
    dk = to_device(keys)
    dv = to_device(vals.reshape(-1)).view(torch.complex128)  # one 16-byte element per key
    ko, vo, r = tb.unique_by_key(dk, dv)
    heads = np.flatnonzero(np.r_[True, keys[1:] != keys[:-1]])
    assert r == heads.size
    assert to_host(ko, np.int32)[:r].tobytes() == keys[heads].tobytes()
    assert to_host(vo.view(torch.float64), np.uint64).reshape(-1, 2)[:r].tobytes() == vals[heads].tobytes()


def test_unique_by_key_known_answer(cuda_device):
    s = json.loads((GOLDEN / "known_answers.json").read_text())["unique_by_key_simple"]
    keys, vals = np.array(s["keys"], dtype=np.int32), np.array(s["values"], dtype=np.int32)
    for inplace in (False, True):
        gk, gv = _unique(keys, vals, inplace)
        assert gk.tolist() == s["out_keys"] and gv.tolist() == s["out_values"]
    assert _unique(keys, None, False)[0].tolist() == s["out_keys"]


def test_unique_float_keys_ieee_equality(cuda_device):
    keys = np.array([0.0, -0.0, 1.5, 1.5, np.nan, np.nan, 2.0, 2.0], dtype=np.float32)
    vals = np.arange(8, dtype=np.int32)
    wk, wv = oracle.port().unique_by_key(keys, vals)
    gk, gv = _unique(keys, vals, False)
    assert gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes()
    assert gv.tolist() == [0, 2, 4, 5, 6]


def test_unique_by_key_one_run_and_all_distinct(cuda_device):
    n = 300001
    gk, gv = _unique(np.full(n, 7, dtype=np.int64), np.arange(n, dtype=np.uint32), True)
    assert gk.tolist() == [7] and gv.tolist() == [0]
    keys = np.arange(n, dtype=np.int32)
    gk, gv = _unique(keys, keys.astype(np.uint32), True)
    assert gk.tobytes() == keys.tobytes() and gv.tobytes() == keys.tobytes()


def test_unique_by_key_unaligned_pointers(cuda_device):
    rng = np.random.default_rng(3)
    n = 70001
    keys = _runs(rng, n, 0.1, np.int32)
    vals = rng.integers(0, 1000, size=n).astype(np.uint32)
    wk, wv = oracle.port().unique_by_key(keys, vals)
    gk, gv = _unique(keys, vals, False, offset=1)
    assert gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes()


@pytest.mark.parametrize("t", ["int8", "uint16", "int32", "uint64", "float32", "float64", "bool"])
def test_select_matches_reference_vectors(cuda_device, t):
    z = np.load(GOLDEN / "reference_vectors.npz")
    k, v = z[f"ubk/{t}/keys"], z[f"ubk/{t}/vals"]
    for inplace in (False, True):
        gk, gv = _unique(k, v, inplace)
        assert gk.tobytes() == z[f"ubk/{t}/out_keys"].tobytes() and gv.tobytes() == z[f"ubk/{t}/out_vals"].tobytes()
    assert _unique(k, None, False)[0].tobytes() == z[f"ubk/{t}/unique"].tobytes()
    out, r = tb.copy_flagged(to_device(v), to_device(z[f"cpf/{t}/flags"]))
    assert to_host(out, v.dtype)[:r].tobytes() == z[f"cpf/{t}/out"].tobytes()


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("fdtype", [np.uint8, np.bool_, np.int32, np.float32, np.int64])
def test_copy_flagged_bit_exact(cuda_device, n, fdtype):
    rng = np.random.default_rng(47 + n)
    chk = oracle.port()
    for p, ddtype in [(0.5, np.uint32), (1 / 16, np.uint64), (1.0, np.uint8), (0.0, np.uint16), (0.9, np.int32)]:
        flags = (rng.random(n) < p).astype(fdtype)
        if np.dtype(fdtype).kind in "iu" and n:
            flags = flags * rng.integers(1, 100, size=n).astype(fdtype)  # any non-zero value selects
        data = rng.integers(0, 250, size=n).astype(ddtype)
        want = chk.copy_flagged(data, flags)
        dd, df = to_device(data), to_device(flags)
        out, r = tb.copy_flagged(dd, df)
        assert r == want.size, (p, ddtype)
        assert to_host(out, data.dtype)[:r].tobytes() == want.tobytes(), (p, ddtype)
        assert to_host(dd, data.dtype).tobytes() == data.tobytes()


def test_copy_flagged_unaligned_and_negative_zero(cuda_device):
    rng = np.random.default_rng(5)
    n = 50001
    data = rng.integers(0, 1 << 31, size=n).astype(np.int32)
    flags = rng.choice(np.array([0.0, -0.0, 1.0, np.nan], dtype=np.float32), size=n)  # -0.0 does not select, NaN does
    want = oracle.port().copy_flagged(data, flags)
    out, r = tb.copy_flagged(to_device(data, offset_elems=3), to_device(flags, offset_elems=1))
    assert r == want.size and to_host(out, np.int32)[:r].tobytes() == want.tobytes()
