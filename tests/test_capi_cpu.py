"""CPU-side checks of the boundary: the shared library loads without a GPU, exports every
symbol the public headers declare, and answers size queries / argument errors."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared(header: Path):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from thrust_b200 import _capi
    names = _declared(ROOT / "include" / "thrust_b200.h")
    assert len(names) >= 25
    for n in names:
        assert hasattr(_capi.lib, n), f"{n} declared in include/ but not exported"
    assert sorted(names) == sorted(_capi.EXPORTS), "the ctypes binding and the header list different entry points"
    # the benchmark generators and the checker are test support: their own library, not the product's
    for n in _declared(ROOT / "thrust_b200" / "datagen" / "datagen.h"):
        assert not hasattr(_capi.lib, n), f"{n} belongs to libtb200_datagen.so, not to the algorithm library"
    assert _capi.lib.tb200_version() >= 100
    assert b"temporary" in _capi.lib.tb200_error_string(_capi.ERR_TEMP_TOO_SMALL)


def test_size_queries_and_argument_errors_need_no_gpu():
    from thrust_b200 import _capi as capi
    need = C.c_size_t(0)
    assert capi.lib.tb200_radix_sort(None, C.byref(need), None, None, 1 << 20, capi.U64, 4, 0, 0, 64, None) == 0
    assert need.value >= (1 << 20) * 12  # alternate key and value buffers live in the scratch
    assert capi.lib.tb200_scan(None, C.byref(need), None, None, 1 << 20, capi.F32, 0, None, None) == 0
    assert 256 <= need.value < (1 << 16)
    assert capi.lib.tb200_scan(None, C.byref(need), None, None, 10, capi.I16, 0, None, None) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_reduce_by_key(None, C.byref(need), None, None, None, None, None, 1 << 20, capi.I32,
                                        capi.F32, None) == 0
    assert capi.lib.tb200_reduce_by_key(None, C.byref(need), None, None, None, None, None, 10, capi.I32,
                                        capi.I8, None) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_radix_sort(None, None, None, None, 10, capi.I32, 0, 0, 0, 32, None) == capi.ERR_INVALID_ARGUMENT


def test_static_scan_refuses_sizes_beyond_its_documented_limits_without_a_gpu():
    from thrust_b200 import _capi as capi
    for dtype, limit in ((capi.F32, 1 << 31), (capi.U32, 1 << 31), (capi.I64, 1 << 29), (capi.F64, 1 << 29)):
        assert capi.lib.tb200_scan_static(None, None, limit + 1, dtype, 0, None, None) == capi.ERR_OVERFLOW
        # at the limit the size check passes (what comes back is an argument or device error)
        assert capi.lib.tb200_scan_static(None, None, limit, dtype, 0, None, None) != capi.ERR_OVERFLOW


def test_python_front_end_refuses_cpu_tensors():
    import torch
    import thrust_b200 as tb
    with pytest.raises(ValueError):
        tb.sort(torch.zeros(4, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        from thrust_b200.sample_sort import ShardedSorter
        ShardedSorter(16, torch.device("cpu"))


def test_host_generators_are_counter_based():
    import numpy as np
    from thrust_b200 import datagen as g
    a = g.host(g.BITS_U64, 1000, 42)
    b = g.host(g.BITS_U64, 500, 42, first=500)
    assert (a[500:] == b).all()
    assert int(a[7]) == g.hash64(42, 7)
    f = g.host(g.UNIFORM_F32, 100000, 7, lo=-1.0, hi=1.0)
    assert f.min() >= -1.0 and f.max() < 1.0 and abs(float(f.mean())) < 0.02
    i = g.host(g.UNIFORM_I64, 100000, 7, lo=-(1 << 20), hi=1 << 20)
    assert i.min() >= -(1 << 20) and i.max() <= (1 << 20)
    h = g.host(g.HEAD_FLAGS_I32, 1 << 18, 11, period=16)
    assert h[0] == 1 and 0.055 < h.mean() < 0.07
    k = g.host(g.AND3_F32, 1 << 18, 4)
    assert not np.isnan(k).any()
    r = g.host(g.ZIPF_RANK_U32, 1 << 16, 5, cdf=g.zipf_cdf())
    assert r.max() < (1 << 16) and (r == 0).mean() > 0.1


def test_argument_validation_precedes_any_device_work():
    """Host-side fault injection: bad scratch is refused before anything touches a GPU."""
    from thrust_b200 import _capi as capi
    need = C.c_size_t(0)
    assert capi.lib.tb200_scan(None, C.byref(need), None, None, 1 << 16, capi.I64, 0, None, None) == 0
    fake = C.c_void_p(0x7f0000000100 + 8)  # never dereferenced: not 256-byte aligned
    assert capi.lib.tb200_scan(fake, C.byref(need), fake, fake, 1 << 16, capi.I64, 0, None, None) == capi.ERR_INVALID_ARGUMENT
    small = C.c_size_t(16)
    fake = C.c_void_p(0x7f0000000100)
    assert capi.lib.tb200_scan(fake, C.byref(small), fake, fake, 1 << 16, capi.I64, 0, None, None) == capi.ERR_TEMP_TOO_SMALL
    assert capi.lib.tb200_reduce_by_key(fake, C.byref(small), fake, fake, fake, fake, fake, 1 << 16, capi.I32, capi.F32,
                                        None) == capi.ERR_TEMP_TOO_SMALL
    assert capi.lib.tb200_partition(None, C.byref(need), None, None, None, None, 10, capi.U64, 4, None, 300, None,
                                    None) == capi.ERR_INVALID_ARGUMENT
    assert capi.lib.tb200_partition(None, C.byref(need), None, None, None, None, 10, capi.F32, 4, None, 3, None,
                                    None) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_gather_segments(None, None, None, None, 17, 8, 0, None, None) == capi.ERR_UNSUPPORTED
    assert capi.lib.tb200_scan_static(None, None, 1 << 40, capi.F32, 0, None, None) == capi.ERR_OVERFLOW


def test_nccl_library_exports_its_entry_point_and_answers_the_size_query():
    import torch  # noqa: F401  (its NCCL is the one the library resolves to)
    from thrust_b200 import _capi as capi, nccl_sort
    names = _declared(ROOT / "include" / "thrust_b200_nccl.h")
    assert names == ["tb200_sample_sort"]
    for n in names:
        assert hasattr(nccl_sort.lib, n) and not hasattr(capi.lib, n), "the NCCL entry lives in its own library"
    push = nccl_sort.temp_bytes(8, 1 << 20, (1 << 20) + (1 << 18), True)
    coll = nccl_sort.temp_bytes(8, 1 << 20, (1 << 20) + (1 << 18), False)
    assert coll >= push + (1 << 20) * 12  # the collective form keeps a partitioned copy of the shard
    need = C.c_size_t(0)
    assert nccl_sort.lib.tb200_sample_sort(None, 3, 2, None, C.byref(need), None, None, 10, None, None, 10, None, None,
                                           None, None) == capi.ERR_INVALID_ARGUMENT  # rank outside the communicator
