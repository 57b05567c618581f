"""Parity of tb200_radix_sort (through the C ABI) with the CPU oracle — bit exact.

Mirrors the reference's sort tests: TestSortSimple / TestSortByKeySimple known answers
(testing/sort.cu:42-76, testing/sort_by_key.cu:44-85), ascending and descending keys of every
arithmetic type over many sizes (testing/sort.cu:80-134), stable sort_by_key with independent
random values so that stability is observable (testing/stable_sort_by_key.cu:99-116), and keys
masked to 0, 3, 6, ... bits, which makes whole digit passes constant
(testing/sort_variable_bits.cu:18-43, testing/sort_by_key_variable_bits.cu:18-50).
"""
import numpy as np
import pytest
import torch

import oracle
import thrust_b200 as tb
from thrust_b200 import _capi as capi
from util import random_keys, to_device, to_host

pytestmark = pytest.mark.gpu

ALL_TYPES = [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64,
             np.float32, np.float64, np.bool_]
SIZES = [0, 1, 2, 3, 31, 32, 33, 255, 1000, 3071, 3072, 3073, 4095, 4096, 4097, 6143, 6144, 6145,
         8191, 8192, 8193, 10027, 10239, 10240, 10241, 65537, 300007]  # incl. tile sizes +-1


@pytest.mark.parametrize("dtype", ALL_TYPES)
def test_sort_keys_all_sizes(cuda_device, dtype):
    chk = oracle.port()
    for n in SIZES:
        rng = np.random.default_rng(1000 + n)
        k = random_keys(rng, n, dtype)
        for desc in (False, True):
            d = to_device(k)
            tb.sort(d, descending=desc)
            assert to_host(d, dtype).tobytes() == chk.sort(k, desc).tobytes(), (n, desc)


@pytest.mark.parametrize("dtype", ALL_TYPES)
def test_stable_sort_by_key_independent_values(cuda_device, dtype):
    chk = oracle.port()
    for n in [0, 1, 2, 33, 1000, 6145, 8193, 10241, 65537, 300007]:
        rng = np.random.default_rng(2000 + n)
        k = random_keys(rng, n, dtype)
        v = rng.integers(0, 1 << 32, size=n, dtype=np.uint32)
        for desc in (False, True):
            dk, dv = to_device(k), to_device(v)
            tb.sort_by_key(dk, dv, descending=desc)
            wk, wv = chk.sort_by_key(k, v, desc)
            assert to_host(dk, dtype).tobytes() == wk.tobytes(), (n, desc)
            assert to_host(dv, np.uint32).tobytes() == wv.tobytes(), (n, desc, "values (stability)")


@pytest.mark.parametrize("dtype", [np.uint8, np.uint16, np.uint32, np.uint64])
def test_sort_variable_bits(cuda_device, dtype):
    chk = oracle.port()
    n = 40009
    for bits in range(0, 8 * np.dtype(dtype).itemsize, 3):
        rng = np.random.default_rng(3000 + bits)
        k = random_keys(rng, n, dtype, bits=bits)
        d = to_device(k)
        tb.sort(d)
        assert to_host(d, dtype).tobytes() == np.sort(k).tobytes(), bits
        dk, dv = to_device(k), to_device(np.arange(n, dtype=np.uint32))
        tb.sort_by_key(dk, dv)
        wk, wv = chk.sort_by_key(k, np.arange(n, dtype=np.uint32))
        assert to_host(dk, dtype).tobytes() == wk.tobytes(), bits
        assert to_host(dv, np.uint32).tobytes() == wv.tobytes(), bits


@pytest.mark.parametrize("vdtype", [np.uint8, np.uint16, np.uint32, np.uint64])
@pytest.mark.parametrize("kdtype", [np.int32, np.uint64, np.float32, np.int16])
def test_sort_by_key_value_widths(cuda_device, kdtype, vdtype):
    rng = np.random.default_rng(4000)
    n = 50021
    k = random_keys(rng, n, kdtype, bits=12)  # many duplicates
    v = rng.integers(0, np.iinfo(vdtype).max, size=n, dtype=vdtype)
    dk, dv = to_device(k), to_device(v)
    tb.sort_by_key(dk, dv)
    wk, wv = oracle.port().sort_by_key(k, v)
    assert to_host(dk, kdtype).tobytes() == wk.tobytes()
    assert to_host(dv, vdtype).tobytes() == wv.tobytes()


def test_sort_by_key_16_byte_values(cuda_device):
    rng = np.random.default_rng(4100)
    n = 30011
    k = random_keys(rng, n, np.uint32, bits=10)
    v = rng.integers(0, 1 << 62, size=(n, 2), dtype=np.uint64)
    dk = to_device(k)
    dv = torch.from_numpy(v.view(np.int64)).to("cuda:0")
    flat = dv.view(-1)
    need = capi.C.c_size_t(0) if hasattr(capi, "C") else None
    import ctypes as C
    need = C.c_size_t(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    capi.check(capi.lib.tb200_radix_sort(None, C.byref(need), None, None, n, capi.U32, 16, 0, 0, 32, stream), "size")
    temp = torch.empty(need.value, dtype=torch.uint8, device="cuda:0")
    capi.check(capi.lib.tb200_radix_sort(C.c_void_p(temp.data_ptr()), C.byref(need), C.c_void_p(dk.data_ptr()),
                                         C.c_void_p(flat.data_ptr()), n, capi.U32, 16, 0, 0, 32, stream), "run")
    capi.check(capi.lib.tb200_temp_status(C.c_void_p(temp.data_ptr()), stream), "status")
    order = np.argsort(k, kind="stable")
    assert to_host(dk, np.uint32).tobytes() == k[order].tobytes()
    assert dv.cpu().numpy().view(np.uint64).tobytes() == v[order].tobytes()


@pytest.mark.parametrize("n", [(1 << 22) + 77, 1 << 24])
def test_sort_many_tiles(cuda_device, n):
    """Long look-back chains: thousands of tiles per pass."""
    rng = np.random.default_rng(5000)
    k = random_keys(rng, n, np.int32)
    d = to_device(k)
    tb.sort(d)
    assert to_host(d, np.int32).tobytes() == np.sort(k).tobytes()
    k64 = random_keys(rng, n // 4, np.uint64)
    v = np.arange(n // 4, dtype=np.uint32)
    dk, dv = to_device(k64), to_device(v)
    tb.sort_by_key(dk, dv)
    order = np.argsort(k64, kind="stable")
    assert to_host(dk, np.uint64).tobytes() == k64[order].tobytes()
    assert to_host(dv, np.uint32).tobytes() == v[order].astype(np.uint32).tobytes()


def test_sort_low_entropy_and_float_specials(cuda_device):
    rng = np.random.default_rng(6000)
    n = 200003
    chk = oracle.port()
    # AND of three words: heavy duplicates, many zeros / subnormals, both signs of zero
    bits = (rng.integers(0, 1 << 32, size=n, dtype=np.uint32) & rng.integers(0, 1 << 32, size=n, dtype=np.uint32)
            & rng.integers(0, 1 << 32, size=n, dtype=np.uint32))
    k = bits.view(np.float32).copy()
    k[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, -np.nan, 1e-45, -1e-45]
    v = np.arange(n, dtype=np.int32)
    for desc in (False, True):
        dk, dv = to_device(k), to_device(v)
        tb.sort_by_key(dk, dv, descending=desc)
        wk, wv = chk.sort_by_key(k, v, desc)
        assert to_host(dk, np.float32).tobytes() == wk.tobytes()
        assert to_host(dv, np.int32).tobytes() == wv.tobytes()
    same = np.full(n, 42, dtype=np.int64)  # every pass is constant: nothing moves
    dk, dv = to_device(same), to_device(v)
    tb.sort_by_key(dk, dv)
    assert to_host(dv, np.int32).tobytes() == v.tobytes()


def test_sort_unaligned_pointers(cuda_device):
    rng = np.random.default_rng(7000)
    n = 70001
    for kdtype in (np.int32, np.uint8, np.uint64):
        k = random_keys(rng, n, kdtype)
        v = rng.integers(0, 1 << 32, size=n, dtype=np.uint32)
        dk, dv = to_device(k, offset_elems=1), to_device(v, offset_elems=3)
        tb.sort_by_key(dk, dv)
        wk, wv = oracle.port().sort_by_key(k, v)
        assert to_host(dk, kdtype).tobytes() == wk.tobytes()
        assert to_host(dv, np.uint32).tobytes() == wv.tobytes()


def test_sort_bit_range(cuda_device):
    rng = np.random.default_rng(8000)
    n = 30011
    k = random_keys(rng, n, np.uint32)
    v = np.arange(n, dtype=np.uint32)
    dk, dv = to_device(k), to_device(v)
    tb.sort_by_key(dk, dv, begin_bit=4, end_bit=15)
    order = np.argsort((k >> 4) & ((1 << 11) - 1), kind="stable")
    assert to_host(dk, np.uint32).tobytes() == k[order].tobytes()
    assert to_host(dv, np.uint32).tobytes() == v[order].tobytes()


def test_sort_known_answers(cuda_device):
    # testing/sort.cu:42-62 and testing/sort_by_key.cu:44-70
    k = np.array([1, 3, 6, 5, 2, 0, 4], dtype=np.int32)
    d = to_device(k)
    tb.sort(d)
    assert to_host(d, np.int32).tolist() == [0, 1, 2, 3, 4, 5, 6]
    dk, dv = to_device(k), to_device(np.arange(7, dtype=np.int32))
    tb.sort_by_key(dk, dv)
    assert to_host(dk, np.int32).tolist() == [0, 1, 2, 3, 4, 5, 6]
    assert to_host(dv, np.int32).tolist() == [5, 0, 4, 1, 6, 3, 2]
    # greater<int>, n = 10027 (testing/sort.cu:92-110)
    rng = np.random.default_rng(9)
    k = rng.integers(-(1 << 31), 1 << 31, size=10027).astype(np.int32)
    d = to_device(k)
    tb.sort(d, descending=True)
    assert to_host(d, np.int32).tobytes() == np.sort(k)[::-1].tobytes()


def test_sort_rejects_bad_arguments(cuda_device):
    import ctypes as C
    need = C.c_size_t(0)
    assert capi.lib.tb200_radix_sort(None, C.byref(need), None, None, 10, 99, 0, 0, 0, 32, None) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_radix_sort(None, C.byref(need), None, None, 10, capi.I32, 3, 0, 0, 32, None) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_radix_sort(None, C.byref(need), None, None, 10, capi.I32, 0, 0, 0, 40, None) == capi.ERR_INVALID_ARGUMENT
    capi.check(capi.lib.tb200_radix_sort(None, C.byref(need), None, None, 1000, capi.I32, 0, 0, 0, 32, None), "size")
    small = C.c_size_t(need.value - 1)
    t = torch.empty(need.value, dtype=torch.uint8, device="cuda:0")
    k = torch.zeros(1000, dtype=torch.int32, device="cuda:0")
    assert capi.lib.tb200_radix_sort(C.c_void_p(t.data_ptr()), C.byref(small), C.c_void_p(k.data_ptr()), None, 1000,
                                     capi.I32, 0, 0, 0, 32, None) == capi.ERR_TEMP_TOO_SMALL


@pytest.mark.parametrize("kdtype,vdtype", [(np.uint64, np.uint32), (np.uint32, None), (np.uint64, np.uint64)])
def test_partition_by_splitters_is_stable(cuda_device, kdtype, vdtype):
    """tb200_partition against a numpy stable partition: bucket b = keys in (s[b-1], s[b]]."""
    import ctypes as C
    rng = np.random.default_rng(4242)
    kcode = capi.U64 if kdtype == np.uint64 else capi.U32
    for n, ns in [(0, 3), (1, 1), (5000, 0), (6144, 7), (100003, 7), (300007, 31), (70001, 255)]:
        k = random_keys(rng, n, kdtype, bits=20 if ns < 100 else None)
        sp = np.sort(random_keys(rng, ns, kdtype, bits=20 if ns < 100 else None))
        v = None if vdtype is None else rng.integers(0, 1 << 31, size=n).astype(vdtype)
        dk, dsp = to_device(k), to_device(sp) if ns else torch.empty(0, dtype=torch.int64, device="cuda:0")
        ok = torch.empty_like(dk)
        dv = to_device(v) if v is not None else None
        ov = torch.empty_like(dv) if dv is not None else None
        counts = torch.zeros(ns + 1, dtype=torch.int64, device="cuda:0")
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        vb = 0 if v is None else v.dtype.itemsize
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_partition(None, C.byref(need), None, None, None, None, n, kcode, vb, None, ns, None,
                                            stream), "size")
        temp = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda:0")
        capi.check(capi.lib.tb200_partition(
            C.c_void_p(temp.data_ptr()), C.byref(need), C.c_void_p(dk.data_ptr()),
            C.c_void_p(dv.data_ptr()) if dv is not None else None, C.c_void_p(ok.data_ptr()),
            C.c_void_p(ov.data_ptr()) if ov is not None else None, n, kcode, vb,
            C.c_void_p(dsp.data_ptr()) if ns else None, ns, C.c_void_p(counts.data_ptr()), stream), "tb200_partition")
        capi.check(capi.lib.tb200_temp_status(C.c_void_p(temp.data_ptr()), stream), "status")
        bucket = np.searchsorted(sp, k, side="left")
        order = np.argsort(bucket, kind="stable")
        assert counts.cpu().numpy().tolist() == np.bincount(bucket, minlength=ns + 1).tolist(), (n, ns)
        assert to_host(ok, kdtype).tobytes() == k[order].tobytes(), (n, ns)
        if v is not None:
            assert to_host(ov, vdtype).tobytes() == v[order].tobytes(), (n, ns)


@pytest.mark.parametrize("kdtype,vdtype", [(np.uint64, np.uint32), (np.uint32, None)])
def test_partition_count_then_scatter_into_separate_buffers(cuda_device, kdtype, vdtype):
    """tb200_partition_count + tb200_partition_scatter: every bucket goes to its own allocation,
    at an odd element offset, and holds its keys in input order (the push form of the exchange)."""
    import ctypes as C
    rng = np.random.default_rng(9001)
    kcode = capi.U64 if kdtype == np.uint64 else capi.U32
    ktorch = torch.int64 if kdtype == np.uint64 else torch.int32
    for n, ns in [(0, 3), (1, 1), (6144, 0), (100003, 7), (250007, 3), (70001, 15)]:
        k = random_keys(rng, n, kdtype, bits=24)
        sp = np.sort(random_keys(rng, ns, kdtype, bits=24))
        v = None if vdtype is None else rng.integers(0, 1 << 31, size=n).astype(vdtype)
        dk = to_device(k)
        dsp = to_device(sp) if ns else torch.empty(0, dtype=ktorch, device="cuda:0")
        dv = to_device(v) if v is not None else None
        counts = torch.zeros(ns + 1, dtype=torch.int64, device="cuda:0")
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        vb = 0 if v is None else v.dtype.itemsize
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_partition_count(None, C.byref(need), None, n, kcode, vb, None, ns, None, stream), "size")
        temp = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda:0")
        capi.check(capi.lib.tb200_partition_count(
            C.c_void_p(temp.data_ptr()), C.byref(need), C.c_void_p(dk.data_ptr()), n, kcode, vb,
            C.c_void_p(dsp.data_ptr()) if ns else None, ns, C.c_void_p(counts.data_ptr()), stream), "count")
        bucket = np.searchsorted(sp, k, side="left")
        want_counts = np.bincount(bucket, minlength=ns + 1).tolist()
        got = counts.cpu().numpy().tolist()
        assert got == want_counts, (n, ns)
        pad = 3  # buckets start three elements into their buffers
        out_k = [torch.full((c + pad + 1,), -1, dtype=ktorch, device="cuda:0") for c in got]
        out_v = [torch.full((c + pad + 1,), -1, dtype=torch.int32, device="cuda:0") for c in got]
        pk = (C.c_void_p * (ns + 1))(*[t.data_ptr() + pad * t.element_size() for t in out_k])
        pv = (C.c_void_p * (ns + 1))(*[t.data_ptr() + pad * 4 for t in out_v])
        capi.check(capi.lib.tb200_partition_scatter(
            C.c_void_p(temp.data_ptr()), C.byref(need), C.c_void_p(dk.data_ptr()),
            C.c_void_p(dv.data_ptr()) if dv is not None else None, n, kcode, vb,
            C.c_void_p(dsp.data_ptr()) if ns else None, ns, pk, pv if vb else None, stream), "scatter")
        capi.check(capi.lib.tb200_temp_status(C.c_void_p(temp.data_ptr()), stream), "status")
        for b in range(ns + 1):
            sel = bucket == b
            hk = to_host(out_k[b], kdtype)
            assert hk[pad:pad + got[b]].tobytes() == k[sel].tobytes(), (n, ns, b)
            assert (hk[:pad] == np.iinfo(kdtype).max).all() and hk[-1] == np.iinfo(kdtype).max, (n, ns, b)
            if v is not None:
                hv = to_host(out_v[b], vdtype)
                assert hv[pad:pad + got[b]].tobytes() == v[sel].tobytes(), (n, ns, b)


@pytest.mark.parametrize("ns", [1, 3, 7, 20])
def test_partition_with_key_index_pairs_divides_equal_keys_in_input_order(cuda_device, ns):
    """The _ties forms: splitters and elements are (key, index) pairs. A handful of distinct keys,
    so most splitter keys repeat; checked against numpy for the one-call form and for count +
    scatter into separate buffers (the push form of the exchange)."""
    import ctypes as C
    rng = np.random.default_rng(31 + ns)
    n, base = 200_003, 5_000_000_000  # indices beyond 32 bits
    k = (rng.integers(0, 3, size=n, dtype=np.uint64) << np.uint64(62)) | np.uint64(0x3fffffffffffffff) * (rng.random(n) < 0.3)
    k = k.astype(np.uint64)  # includes the largest key, which is also the value of the tile padding
    v = rng.integers(0, 1 << 31, size=n).astype(np.uint32)
    cand = np.sort(rng.choice(n, size=ns, replace=False))
    order = np.lexsort((cand, k[cand]))
    sp, si = k[cand][order], (cand[order] + base).astype(np.int64)
    g = np.arange(n, dtype=np.int64) + base
    bucket = ((sp[None, :] < k[:, None]) | ((sp[None, :] == k[:, None]) & (si[None, :] < g[:, None]))).sum(axis=1)
    want_counts = np.bincount(bucket, minlength=ns + 1).tolist()
    perm = np.argsort(bucket, kind="stable")
    dk, dv, dsp, dsi = to_device(k), to_device(v), to_device(sp), to_device(si)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = C.c_size_t(0)
    capi.check(capi.lib.tb200_partition_ties(None, C.byref(need), None, None, None, None, n, capi.U64, 4, None, None, ns,
                                             base, None, stream), "size")
    temp = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda:0")
    ok, ov = torch.empty_like(dk), torch.empty_like(dv)
    counts = torch.zeros(ns + 1, dtype=torch.int64, device="cuda:0")
    P = lambda t: C.c_void_p(t.data_ptr())
    capi.check(capi.lib.tb200_partition_ties(P(temp), C.byref(need), P(dk), P(dv), P(ok), P(ov), n, capi.U64, 4, P(dsp),
                                             P(dsi), ns, base, P(counts), stream), "tb200_partition_ties")
    capi.check(capi.lib.tb200_temp_status(P(temp), stream), "status")
    assert counts.cpu().numpy().tolist() == want_counts
    assert to_host(ok, np.uint64).tobytes() == k[perm].tobytes() and to_host(ov, np.uint32).tobytes() == v[perm].tobytes()
    counts.zero_()
    capi.check(capi.lib.tb200_partition_count_ties(P(temp), C.byref(need), P(dk), n, capi.U64, 4, P(dsp), P(dsi), ns, base,
                                                   P(counts), stream), "count")
    got = counts.cpu().numpy().tolist()
    assert got == want_counts
    out_k = [torch.full((c + 1,), -1, dtype=torch.int64, device="cuda:0") for c in got]
    out_v = [torch.full((c + 1,), -1, dtype=torch.int32, device="cuda:0") for c in got]
    pk = (C.c_void_p * (ns + 1))(*[t.data_ptr() for t in out_k])
    pv = (C.c_void_p * (ns + 1))(*[t.data_ptr() for t in out_v])
    capi.check(capi.lib.tb200_partition_scatter_ties(P(temp), C.byref(need), P(dk), P(dv), n, capi.U64, 4, P(dsp), P(dsi),
                                                     ns, base, pk, pv, stream), "scatter")
    capi.check(capi.lib.tb200_temp_status(P(temp), stream), "status")
    for b in range(ns + 1):
        sel = bucket == b
        assert to_host(out_k[b], np.uint64)[:got[b]].tobytes() == k[sel].tobytes(), b
        assert to_host(out_v[b], np.uint32)[:got[b]].tobytes() == v[sel].tobytes(), b


@pytest.mark.parametrize("dtype", [np.uint64, np.uint32])
def test_gather_segments_concatenates_ranges(cuda_device, dtype):
    """tb200_gather_segments on local pointers: odd offsets and lengths, empty segments."""
    import ctypes as C
    rng = np.random.default_rng(77)
    srcs = [rng.integers(0, 1 << 31, size=m).astype(dtype) for m in (100003, 5, 70001, 1 << 16)]
    devs = [to_device(a, offset_elems=i % 2) for i, a in enumerate(srcs)]
    offs = [3, 0, 12345, 1]
    cnts = [99999, 0, 40001, (1 << 16) - 1]
    want = np.concatenate([a[o:o + c] for a, o, c in zip(srcs, offs, cnts)])
    dst = torch.zeros(want.size + 1, dtype=torch.int64 if dtype == np.uint64 else torch.int32, device="cuda:0")[1:]
    g = len(srcs)
    ptrs = (C.c_void_p * g)(*[d.data_ptr() for d in devs])
    o = (C.c_uint64 * g)(*offs)
    c = (C.c_uint64 * g)(*cnts)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    capi.check(capi.lib.tb200_gather_segments(C.c_void_p(dst.data_ptr()), ptrs, o, c, g, np.dtype(dtype).itemsize, 3,
                                              None, stream), "tb200_gather_segments")
    torch.cuda.synchronize()
    assert to_host(dst, dtype).tobytes() == want.tobytes()


def test_gather_that_counts_digits_then_sort_finish(cuda_device):
    """tb200_radix_sort_begin + gather with digit counting + tb200_radix_sort_finish == tb200_radix_sort."""
    import ctypes as C
    rng = np.random.default_rng(78)
    parts_k = [random_keys(rng, m, np.uint64) for m in (70001, 3, 123457)]
    parts_v = [rng.integers(0, 1 << 32, size=a.size, dtype=np.uint32) for a in parts_k]
    dk = [to_device(a, offset_elems=1) for a in parts_k]
    dv = [to_device(a, offset_elems=3) for a in parts_v]
    n = sum(a.size for a in parts_k)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = C.c_size_t(0)
    capi.check(capi.lib.tb200_radix_sort(None, C.byref(need), None, None, n, capi.U64, 4, 0, 0, 64, stream), "size")
    temp = torch.empty(need.value, dtype=torch.uint8, device="cuda:0")
    out_k = torch.empty(n, dtype=torch.int64, device="cuda:0")
    out_v = torch.empty(n, dtype=torch.int32, device="cuda:0")
    g = 3
    zeros = (C.c_uint64 * g)(0, 0, 0)
    cnts = (C.c_uint64 * g)(*[a.size for a in parts_k])
    capi.check(capi.lib.tb200_radix_sort_begin(C.c_void_p(temp.data_ptr()), C.byref(need), n, capi.U64, 4, stream), "begin")
    capi.check(capi.lib.tb200_gather_segments(C.c_void_p(out_k.data_ptr()), (C.c_void_p * g)(*[d.data_ptr() for d in dk]),
                                              zeros, cnts, g, 8, 1, C.c_void_p(temp.data_ptr()), stream), "gather keys")
    capi.check(capi.lib.tb200_gather_segments(C.c_void_p(out_v.data_ptr()), (C.c_void_p * g)(*[d.data_ptr() for d in dv]),
                                              zeros, cnts, g, 4, 1, None, stream), "gather values")
    capi.check(capi.lib.tb200_radix_sort_finish(C.c_void_p(temp.data_ptr()), C.byref(need), C.c_void_p(out_k.data_ptr()),
                                                C.c_void_p(out_v.data_ptr()), n, capi.U64, 4, stream), "finish")
    capi.check(capi.lib.tb200_temp_status(C.c_void_p(temp.data_ptr()), stream), "status")
    wk, wv = oracle.port().sort_by_key(np.concatenate(parts_k), np.concatenate(parts_v))
    assert to_host(out_k, np.uint64).tobytes() == wk.tobytes()
    assert to_host(out_v, np.uint32).tobytes() == wv.tobytes()


def test_sort_more_than_2_pow_30_keys(cuda_device):
    """n > 2^30 switches the look-back descriptors and output indices to 64 bits."""
    from thrust_b200 import datagen as g
    n = (1 << 30) + 12345
    k = g.device(g.BITS_U32, n, 99, dev=cuda_device)  # int32 tensor holding uint32 bit patterns
    before_sum = int(k.view(torch.int32).sum(dtype=torch.int64))
    before_xor = 0
    for s in range(0, n, 1 << 28):  # xor checksum in chunks (bitwise ops keep int32)
        c = k[s:s + (1 << 28)]
        while c.numel() > 1:
            h = c.numel() // 2
            c = torch.cat([c[:h] ^ c[h:2 * h], c[2 * h:]])
        before_xor ^= int(c.item())
    tb.sort(k, key_dtype=capi.U32)
    u = k.view(torch.int32)
    # unsigned order: compare after flipping the sign bit, chunk by chunk
    ok = True
    for s in range(0, n - 1, 1 << 28):
        e = min(n, s + (1 << 28) + 1)
        f = u[s:e] ^ (-2147483648)
        ok = ok and bool((f[1:] >= f[:-1]).all())
    assert ok
    assert int(u.sum(dtype=torch.int64)) == before_sum
    after_xor = 0
    for s in range(0, n, 1 << 28):
        c = k[s:s + (1 << 28)]
        while c.numel() > 1:
            h = c.numel() // 2
            c = torch.cat([c[:h] ^ c[h:2 * h], c[2 * h:]])
        after_xor ^= int(c.item())
    assert after_xor == before_xor
