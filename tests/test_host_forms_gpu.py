"""Parity of the host-buffer entry points (tb200_radix_sort_host, tb200_scan_host,
tb200_reduce_by_key_host) with the CPU oracle.

These replace the reference's flagship usage — host vector -> device vector -> algorithm -> host
(README.md:42-54; the copies are thrust/system/cuda/detail/internal/copy_cross_system.h:51-113) —
so they are given plain numpy arrays (pageable memory) as well as pinned torch tensors. Keys,
values, stability and run counts are compared bit for bit; floating-point sums within 1e-5 of the
sum of absolute values.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from thrust_b200 import _capi as capi

pytestmark = pytest.mark.gpu

_DT = {np.dtype(np.int8): capi.I8, np.dtype(np.uint8): capi.U8, np.dtype(np.int16): capi.I16,
       np.dtype(np.uint16): capi.U16, np.dtype(np.int32): capi.I32, np.dtype(np.uint32): capi.U32,
       np.dtype(np.int64): capi.I64, np.dtype(np.uint64): capi.U64, np.dtype(np.float32): capi.F32,
       np.dtype(np.float64): capi.F64}


def _host_copy(a: np.ndarray, pinned: bool):
    """(numpy view the C call writes into, object that keeps the memory alive)."""
    if not pinned:
        b = np.ascontiguousarray(a).copy()
        return b, b
    t = torch.empty(max(a.nbytes, 1), dtype=torch.uint8).pin_memory()
    view = t.numpy()[:a.nbytes].view(a.dtype)
    view[...] = a
    return view, t


def _ptr(a: np.ndarray):
    return C.c_void_p(a.ctypes.data) if a.size else None


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("n", [0, 1, 5, 6143, 6144, 6145, 100003, (1 << 20) + 77])
def test_radix_sort_host_pairs_u64_u32(cuda_device, n, pinned):
    rng = np.random.default_rng(n + 1)
    keys = rng.integers(0, 1 << 12, size=n, dtype=np.uint64) << np.uint64(40)  # heavy duplicates: stability shows
    vals = np.arange(n, dtype=np.uint32)
    wk, wv = oracle.port().sort_by_key(keys, vals)
    hk, keep_k = _host_copy(keys, pinned)
    hv, keep_v = _host_copy(vals, pinned)
    rc = capi.lib.tb200_radix_sort_host(_ptr(hk), _ptr(hv), n, capi.U64, 4, 0, _stream(cuda_device))
    capi.check(rc, "tb200_radix_sort_host")
    assert hk.tobytes() == wk.tobytes()
    assert hv.tobytes() == wv.tobytes()


@pytest.mark.parametrize("dtype,val_dtype,descending", [
    (np.int32, None, False), (np.int32, None, True), (np.float32, np.int32, False), (np.float64, np.uint8, True),
    (np.int8, np.uint16, False), (np.uint16, np.uint64, False), (np.int64, np.int64, True),
])
def test_radix_sort_host_other_types(cuda_device, dtype, val_dtype, descending):
    rng = np.random.default_rng(7)
    n = 70001
    u = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[np.dtype(dtype).itemsize]
    keys = rng.integers(0, np.iinfo(u).max, size=n, dtype=u, endpoint=True).view(dtype)  # floats: all bit patterns
    chk = oracle.port()
    hk, _k = _host_copy(keys, False)
    if val_dtype is None:
        want = chk.sort(keys, descending)
        capi.check(capi.lib.tb200_radix_sort_host(_ptr(hk), None, n, _DT[np.dtype(dtype)], 0, int(descending),
                                                  _stream(cuda_device)), "tb200_radix_sort_host")
        assert hk.tobytes() == want.tobytes()
        return
    vals = rng.integers(0, 100, size=n).astype(val_dtype)
    wk, wv = chk.sort_by_key(keys, vals, descending)
    hv, _v = _host_copy(vals, False)
    capi.check(capi.lib.tb200_radix_sort_host(_ptr(hk), _ptr(hv), n, _DT[np.dtype(dtype)], hv.dtype.itemsize,
                                              int(descending), _stream(cuda_device)), "tb200_radix_sort_host")
    assert hk.tobytes() == wk.tobytes()
    assert hv.tobytes() == wv.tobytes()


@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("dtype", [np.int32, np.uint64, np.float32, np.float64])
@pytest.mark.parametrize("exclusive", [0, 1])
def test_scan_host(cuda_device, dtype, exclusive, pinned):
    rng = np.random.default_rng(31)
    chk = oracle.port()
    for n in (0, 1, 10241, 300007):
        if np.dtype(dtype).kind == "f":
            a = rng.uniform(-1, 1, size=n).astype(dtype)
        else:
            a = rng.integers(0, 1 << 20, size=n).astype(dtype)
        init = np.array([3], dtype=dtype)
        want = chk.scan(a, bool(exclusive), init[0] if exclusive else None)
        hin, _i = _host_copy(a, pinned)
        hout, _o = _host_copy(np.zeros_like(a), pinned)
        rc = capi.lib.tb200_scan_host(_ptr(hin), _ptr(hout), n, _DT[np.dtype(dtype)], exclusive,
                                      _ptr(init) if exclusive else None, _stream(cuda_device))
        capi.check(rc, "tb200_scan_host")
        assert hin.tobytes() == a.tobytes()  # the input is not modified
        if np.dtype(dtype).kind == "f":
            tol = 1e-5 * float(np.abs(a.astype(np.float64)).sum()) + 1e-30
            assert n == 0 or float(np.max(np.abs(hout.astype(np.float64) - want.astype(np.float64)))) <= tol
        else:
            assert hout.tobytes() == want.tobytes()


@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("kdtype,vdtype", [(np.int32, np.int32), (np.uint64, np.int64), (np.uint8, np.uint32),
                                           (np.int32, np.float32)])
def test_reduce_by_key_host(cuda_device, kdtype, vdtype, pinned):
    rng = np.random.default_rng(12)
    chk = oracle.port()
    for n in (0, 1, 6401, 250007):
        ids = np.cumsum(rng.random(n) < 1 / 16)
        keys = (ids % 2 if np.dtype(kdtype).itemsize == 1 else ids).astype(kdtype)
        if np.dtype(vdtype).kind == "f":
            vals = rng.uniform(-50, 50, size=n).astype(vdtype)
        else:
            vals = rng.integers(0, 1 << 20, size=n).astype(vdtype)
        wk, wv = chk.reduce_by_key(keys, vals)
        hk, _a = _host_copy(keys, pinned)
        hv, _b = _host_copy(vals, pinned)
        ok, _c = _host_copy(np.zeros_like(keys), pinned)
        ov, _d = _host_copy(np.zeros_like(vals), pinned)
        runs = C.c_uint64(12345)
        rc = capi.lib.tb200_reduce_by_key_host(_ptr(hk), _ptr(hv), _ptr(ok), _ptr(ov), C.byref(runs), n,
                                               _DT[np.dtype(kdtype)], _DT[np.dtype(vdtype)], _stream(cuda_device))
        capi.check(rc, "tb200_reduce_by_key_host")
        r = int(runs.value)
        assert r == wk.size
        assert ok[:r].tobytes() == wk.tobytes()
        if np.dtype(vdtype).kind == "f" and n:
            heads = np.flatnonzero(np.r_[True, keys[1:] != keys[:-1]])
            abs_sums = np.add.reduceat(np.abs(vals.astype(np.float64)), heads)
            assert np.all(np.abs(ov[:r].astype(np.float64) - wv.astype(np.float64)) <= 1e-5 * abs_sums + 1e-30)
        else:
            assert ov[:r].tobytes() == wv.tobytes()


def test_host_forms_reject_bad_arguments(cuda_device):
    st = _stream(cuda_device)
    one = np.zeros(4, dtype=np.int32)
    assert capi.lib.tb200_radix_sort_host(None, None, 4, capi.I32, 0, 0, st) == capi.ERR_INVALID_ARGUMENT
    assert capi.lib.tb200_radix_sort_host(_ptr(one), None, 4, capi.I32, 4, 0, st) == capi.ERR_INVALID_ARGUMENT
    assert capi.lib.tb200_radix_sort_host(_ptr(one), None, 4, 99, 0, 0, st) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_scan_host(None, _ptr(one), 4, capi.I32, 0, None, st) == capi.ERR_INVALID_ARGUMENT
    assert capi.lib.tb200_scan_host(_ptr(one), _ptr(one), 4, capi.I16, 0, None, st) == capi.ERR_UNSUPPORTED
    runs = C.c_uint64(0)
    assert capi.lib.tb200_reduce_by_key_host(_ptr(one), _ptr(one), _ptr(one), None, C.byref(runs), 4, capi.I32,
                                             capi.I32, st) == capi.ERR_INVALID_ARGUMENT
