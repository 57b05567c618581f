"""Python mirror of the thrust:: algorithms this library replaces.

Each function takes CUDA tensors, passes their device pointers and the current
stream through the C ABI and, like the reference's default ``thrust::cuda::par``
policy, synchronises and checks the device status before returning
(thrust/system/cuda/detail/util.h:113-140) unless ``sync=False``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _capi as capi

_TORCH_TO_TB = {
    torch.int8: capi.I8, torch.uint8: capi.U8, torch.int16: capi.I16, torch.uint16: capi.U16,
    torch.int32: capi.I32, torch.uint32: capi.U32, torch.int64: capi.I64, torch.uint64: capi.U64,
    torch.float32: capi.F32, torch.float64: capi.F64, torch.bool: capi.BOOL,
}
_NUMERIC = (capi.I32, capi.U32, capi.I64, capi.U64, capi.F32, capi.F64)


def tb200_dtype(t: torch.Tensor, dtype: Optional[int] = None) -> int:
    """tb200_dtype code of a tensor (``dtype`` overrides, e.g. to read int64 storage as U64)."""
    if dtype is not None:
        if capi.DTYPE_BYTES[dtype] != t.element_size():
            raise ValueError("dtype override must keep the element size")
        return dtype
    try:
        return _TORCH_TO_TB[t.dtype]
    except KeyError:
        raise TypeError(f"no tb200 dtype for {t.dtype}") from None


def _check_tensor(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (thrust_b200 has no CPU path)")
    if not t.is_contiguous() or t.dim() != 1:
        raise ValueError(f"{name} must be a contiguous 1-D tensor")


def _stream(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _temp(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _finish(temp: torch.Tensor, stream, what: str, sync: bool) -> None:
    if sync:
        capi.check(capi.lib.tb200_temp_status(C.c_void_p(temp.data_ptr()), stream), what)


def sort_by_key(keys: torch.Tensor, values: Optional[torch.Tensor] = None, descending: bool = False,
                key_dtype: Optional[int] = None, begin_bit: int = 0, end_bit: Optional[int] = None,
                sync: bool = True, temp: Optional[torch.Tensor] = None) -> None:
    """thrust::sort_by_key / stable_sort_by_key (thrust/sort.h), in place; values=None sorts keys only."""
    _check_tensor(keys, "keys")
    kd = tb200_dtype(keys, key_dtype)
    n = keys.numel()
    vb = 0
    vptr = None
    if values is not None:
        _check_tensor(values, "values")
        if values.numel() != n:
            raise ValueError("keys and values differ in length")
        vb = values.element_size()
        vptr = values.data_ptr()
    if end_bit is None:
        end_bit = 8 * keys.element_size()
    with torch.cuda.device(keys.device):
        stream = _stream(keys)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_radix_sort(None, C.byref(need), None, None, n, kd, vb, int(descending),
                                             begin_bit, end_bit, stream), "tb200_radix_sort(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, keys.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_radix_sort(C.c_void_p(temp.data_ptr()), C.byref(have),
                                             C.c_void_p(keys.data_ptr()), C.c_void_p(vptr), n, kd, vb,
                                             int(descending), begin_bit, end_bit, stream), "tb200_radix_sort")
        _finish(temp, stream, "tb200_radix_sort", sync)


def sort(keys: torch.Tensor, descending: bool = False, **kw) -> None:
    """thrust::sort on arithmetic keys (stable on this path, like the reference's radix path)."""
    sort_by_key(keys, None, descending, **kw)


stable_sort = sort
stable_sort_by_key = sort_by_key


def _scan(inp: torch.Tensor, out: Optional[torch.Tensor], exclusive: bool, init, dtype: Optional[int],
          sync: bool, temp: Optional[torch.Tensor]) -> torch.Tensor:
    _check_tensor(inp, "input")
    dt = tb200_dtype(inp, dtype)
    if dt not in _NUMERIC:
        raise TypeError("scan supports 4- and 8-byte integers, float32 and float64")
    if out is None:
        out = torch.empty_like(inp)
    _check_tensor(out, "output")
    if out.numel() != inp.numel() or out.element_size() != inp.element_size():
        raise ValueError("output must match the input")
    n = inp.numel()
    init_buf = None
    if init is not None:
        ctype = {capi.I32: C.c_int32, capi.U32: C.c_uint32, capi.I64: C.c_int64, capi.U64: C.c_uint64,
                 capi.F32: C.c_float, capi.F64: C.c_double}[dt]
        init_buf = ctype(init)
    with torch.cuda.device(inp.device):
        stream = _stream(inp)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_scan(None, C.byref(need), None, None, n, dt, int(exclusive), None, stream),
                   "tb200_scan(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, inp.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_scan(C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(inp.data_ptr()),
                                       C.c_void_p(out.data_ptr()), n, dt, int(exclusive),
                                       C.byref(init_buf) if init_buf is not None else None, stream),
                   "tb200_scan")
        _finish(temp, stream, "tb200_scan", sync)
    return out


def inclusive_scan(inp: torch.Tensor, out: Optional[torch.Tensor] = None, dtype: Optional[int] = None,
                   sync: bool = True, temp: Optional[torch.Tensor] = None, init=None) -> torch.Tensor:
    """thrust::inclusive_scan with plus (thrust/scan.h:99); ``out`` may be ``inp``. ``init`` seeds the
    scan (out[i] = init + in[0] + ... + in[i]); None is the plain form."""
    return _scan(inp, out, False, init, dtype, sync, temp)


def exclusive_scan(inp: torch.Tensor, out: Optional[torch.Tensor] = None, init=None,
                   dtype: Optional[int] = None, sync: bool = True,
                   temp: Optional[torch.Tensor] = None) -> torch.Tensor:
    """thrust::exclusive_scan with plus; init=None is the value-initialised default."""
    return _scan(inp, out, True, init, dtype, sync, temp)


def reduce(inp: torch.Tensor, init=None, dtype: Optional[int] = None, out: Optional[torch.Tensor] = None,
           temp: Optional[torch.Tensor] = None):
    """thrust::reduce with plus (thrust/reduce.h; cuda/detail/reduce.h:1029-1062): init + the sum of
    ``inp`` in the element type (integers wrap). Returns a Python number; like the reference it
    synchronises to read the result back (cuda/detail/reduce.h:984-1000)."""
    _check_tensor(inp, "input")
    dt = tb200_dtype(inp, dtype)
    ctypes_of = {capi.I8: C.c_int8, capi.U8: C.c_uint8, capi.I16: C.c_int16, capi.U16: C.c_uint16,
                 capi.I32: C.c_int32, capi.U32: C.c_uint32, capi.I64: C.c_int64, capi.U64: C.c_uint64,
                 capi.F32: C.c_float, capi.F64: C.c_double}
    if dt not in ctypes_of:
        raise TypeError("reduce supports integers of 1 to 8 bytes, float32 and float64")
    ctype = ctypes_of[dt]
    init_buf = ctype(init) if init is not None else None
    n = inp.numel()
    if out is None:
        out = torch.empty(16, dtype=torch.uint8, device=inp.device)
    with torch.cuda.device(inp.device):
        stream = _stream(inp)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_reduce(None, C.byref(need), None, n, dt, None, None, stream), "tb200_reduce(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, inp.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_reduce(C.c_void_p(temp.data_ptr()), C.byref(have),
                                         C.c_void_p(inp.data_ptr()) if n else None, n, dt,
                                         C.byref(init_buf) if init_buf is not None else None,
                                         C.c_void_p(out.data_ptr()), stream), "tb200_reduce")
        _finish(temp, stream, "tb200_reduce", True)
    raw = bytes(out.view(torch.uint8)[:C.sizeof(ctype)].cpu().numpy().tobytes())
    return ctype.from_buffer_copy(raw).value


def _scan_by_key(keys: torch.Tensor, values: torch.Tensor, out: Optional[torch.Tensor], exclusive: bool, init,
                 key_dtype: Optional[int], val_dtype: Optional[int], sync: bool,
                 temp: Optional[torch.Tensor]) -> torch.Tensor:
    _check_tensor(keys, "keys")
    _check_tensor(values, "values")
    n = keys.numel()
    if values.numel() != n:
        raise ValueError("keys and values differ in length")
    kd = tb200_dtype(keys, key_dtype)
    vd = tb200_dtype(values, val_dtype)
    if vd not in _NUMERIC:
        raise TypeError("scan_by_key supports 4- and 8-byte integer, float32 and float64 values")
    if out is None:
        out = torch.empty_like(values)
    _check_tensor(out, "output")
    if out.numel() != n or out.element_size() != values.element_size():
        raise ValueError("output must match the values")
    init_buf = None
    if exclusive and init is not None:
        ctype = {capi.I32: C.c_int32, capi.U32: C.c_uint32, capi.I64: C.c_int64, capi.U64: C.c_uint64,
                 capi.F32: C.c_float, capi.F64: C.c_double}[vd]
        init_buf = ctype(init)
    with torch.cuda.device(keys.device):
        stream = _stream(keys)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_scan_by_key(None, C.byref(need), None, None, None, n, kd, vd, int(exclusive), None,
                                              stream), "tb200_scan_by_key(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, keys.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_scan_by_key(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), C.c_void_p(values.data_ptr()),
            C.c_void_p(out.data_ptr()), n, kd, vd, int(exclusive),
            C.byref(init_buf) if init_buf is not None else None, stream), "tb200_scan_by_key")
        _finish(temp, stream, "tb200_scan_by_key", sync)
    return out


def inclusive_scan_by_key(keys: torch.Tensor, values: torch.Tensor, out: Optional[torch.Tensor] = None,
                          key_dtype: Optional[int] = None, val_dtype: Optional[int] = None, sync: bool = True,
                          temp: Optional[torch.Tensor] = None) -> torch.Tensor:
    """thrust::inclusive_scan_by_key (equal_to, plus); ``out`` may be ``values``."""
    return _scan_by_key(keys, values, out, False, None, key_dtype, val_dtype, sync, temp)


def exclusive_scan_by_key(keys: torch.Tensor, values: torch.Tensor, out: Optional[torch.Tensor] = None, init=None,
                          key_dtype: Optional[int] = None, val_dtype: Optional[int] = None, sync: bool = True,
                          temp: Optional[torch.Tensor] = None) -> torch.Tensor:
    """thrust::exclusive_scan_by_key (equal_to, plus): every run restarts at ``init`` (default 0)."""
    return _scan_by_key(keys, values, out, True, init, key_dtype, val_dtype, sync, temp)


def reduce_by_key(keys: torch.Tensor, values: torch.Tensor, keys_out: Optional[torch.Tensor] = None,
                  values_out: Optional[torch.Tensor] = None, key_dtype: Optional[int] = None,
                  val_dtype: Optional[int] = None,
                  temp: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """thrust::reduce_by_key (equal_to, plus). Returns (keys_out, values_out, number of runs);
    like the reference it synchronises to read the run count (cuda/detail/reduce_by_key.h:1049-1052)."""
    _check_tensor(keys, "keys")
    _check_tensor(values, "values")
    n = keys.numel()
    if values.numel() != n:
        raise ValueError("keys and values differ in length")
    kd = tb200_dtype(keys, key_dtype)
    vd = tb200_dtype(values, val_dtype)
    if keys_out is None:
        keys_out = torch.empty_like(keys)
    if values_out is None:
        values_out = torch.empty_like(values)
    with torch.cuda.device(keys.device):
        stream = _stream(keys)
        runs = torch.zeros(1, dtype=torch.int64, device=keys.device)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_reduce_by_key(None, C.byref(need), None, None, None, None, None, n, kd, vd,
                                                stream), "tb200_reduce_by_key(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, keys.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_reduce_by_key(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()),
            C.c_void_p(values.data_ptr()), C.c_void_p(keys_out.data_ptr()), C.c_void_p(values_out.data_ptr()),
            C.c_void_p(runs.data_ptr()), n, kd, vd, stream), "tb200_reduce_by_key")
        _finish(temp, stream, "tb200_reduce_by_key", True)
        return keys_out, values_out, int(runs.item())


def unique_by_key(keys: torch.Tensor, values: Optional[torch.Tensor] = None, keys_out: Optional[torch.Tensor] = None,
                  values_out: Optional[torch.Tensor] = None, key_dtype: Optional[int] = None, inplace: bool = False,
                  temp: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor], int]:
    """thrust::unique_by_key_copy (thrust/unique.h): the first (key, value) of every run of equal
    consecutive keys. values=None is thrust::unique_copy; inplace=True compacts the inputs
    themselves (thrust::unique_by_key / thrust::unique). Returns (keys_out, values_out, count);
    synchronises to read the count like the reference (cuda/detail/unique_by_key.h:789-791)."""
    _check_tensor(keys, "keys")
    n = keys.numel()
    kd = tb200_dtype(keys, key_dtype)
    vb = 0
    if values is not None:
        _check_tensor(values, "values")
        if values.numel() != n:
            raise ValueError("keys and values differ in length")
        vb = values.element_size()
    if inplace:
        keys_out, values_out = keys, values
    else:
        if keys_out is None:
            keys_out = torch.empty_like(keys)
        if values is not None and values_out is None:
            values_out = torch.empty_like(values)
    with torch.cuda.device(keys.device):
        stream = _stream(keys)
        count = torch.zeros(1, dtype=torch.int64, device=keys.device)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_unique_by_key(None, C.byref(need), None, None, None, None, None, n, kd, vb, stream),
                   "tb200_unique_by_key(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, keys.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_unique_by_key(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()),
            C.c_void_p(values.data_ptr()) if values is not None else None, C.c_void_p(keys_out.data_ptr()),
            C.c_void_p(values_out.data_ptr()) if values_out is not None else None, C.c_void_p(count.data_ptr()), n, kd,
            vb, stream), "tb200_unique_by_key")
        _finish(temp, stream, "tb200_unique_by_key", True)
        return keys_out, values_out, int(count.item())


def unique(keys: torch.Tensor, out: Optional[torch.Tensor] = None, key_dtype: Optional[int] = None,
           inplace: bool = False) -> Tuple[torch.Tensor, int]:
    """thrust::unique_copy / thrust::unique (inplace=True) with equal_to."""
    k, _, r = unique_by_key(keys, None, out, None, key_dtype, inplace)
    return k, r


def copy_flagged(data: torch.Tensor, flags: torch.Tensor, out: Optional[torch.Tensor] = None,
                 flag_dtype: Optional[int] = None, temp: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, int]:
    """thrust::copy_if(first, last, stencil, result, thrust::identity<Flag>()) (thrust/copy.h): the
    elements whose flag is non-zero, in input order. Returns (out, count); synchronises to read the
    count like the reference (cuda/detail/copy_if.h:771-773)."""
    _check_tensor(data, "data")
    _check_tensor(flags, "flags")
    n = data.numel()
    if flags.numel() != n:
        raise ValueError("data and flags differ in length")
    fd = tb200_dtype(flags, flag_dtype)
    if out is None:
        out = torch.empty_like(data)
    _check_tensor(out, "out")
    with torch.cuda.device(data.device):
        stream = _stream(data)
        count = torch.zeros(1, dtype=torch.int64, device=data.device)
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_copy_flagged(None, C.byref(need), None, None, None, None, n, data.element_size(), fd,
                                               stream), "tb200_copy_flagged(size)")
        if temp is None or temp.numel() < need.value:
            temp = _temp(need.value, data.device)
        have = C.c_size_t(temp.numel())
        capi.check(capi.lib.tb200_copy_flagged(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(data.data_ptr()), C.c_void_p(flags.data_ptr()),
            C.c_void_p(out.data_ptr()), C.c_void_p(count.data_ptr()), n, data.element_size(), fd, stream),
            "tb200_copy_flagged")
        _finish(temp, stream, "tb200_copy_flagged", True)
        return out, int(count.item())


def histogram_sorted(sorted_data: torch.Tensor, bin_values: torch.Tensor, dtype: Optional[int] = None,
                     sync: bool = True) -> torch.Tensor:
    """upper_bound of every bin value in sorted data + adjacent_difference (examples/histogram.cu:84-97)."""
    _check_tensor(sorted_data, "sorted_data")
    _check_tensor(bin_values, "bin_values")
    dt = tb200_dtype(sorted_data, dtype)
    counts = torch.empty(bin_values.numel(), dtype=torch.int32, device=sorted_data.device)
    with torch.cuda.device(sorted_data.device):
        stream = _stream(sorted_data)
        capi.check(capi.lib.tb200_histogram_sorted(C.c_void_p(sorted_data.data_ptr()), sorted_data.numel(), dt,
                                                   C.c_void_p(bin_values.data_ptr()), bin_values.numel(),
                                                   C.c_void_p(counts.data_ptr()), stream),
                   "tb200_histogram_sorted")
        if sync:
            torch.cuda.current_stream(sorted_data.device).synchronize()
    return counts


def dense_histogram(data: torch.Tensor, bin_values: torch.Tensor, dtype: Optional[int] = None) -> torch.Tensor:
    """The whole dense-histogram recipe of examples/histogram.cu:60-101: copy, sort, search, difference."""
    work = data.clone()
    sort(work, key_dtype=dtype)
    return histogram_sorted(work, bin_values, dtype)
