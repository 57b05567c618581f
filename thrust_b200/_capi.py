"""ctypes binding of libthrust_b200.so (the C ABI declared in include/thrust_b200.h).

There is no fallback: if the CUDA library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libthrust_b200.so"

# tb200_dtype
I8, U8, I16, U16, I32, U32, I64, U64, F32, F64, BOOL = range(11)
DTYPE_BYTES = {I8: 1, U8: 1, I16: 2, U16: 2, I32: 4, U32: 4, I64: 8, U64: 8, F32: 4, F64: 8, BOOL: 1}

OK = 0
ERR_UNSUPPORTED, ERR_INVALID_ARGUMENT, ERR_TEMP_TOO_SMALL, ERR_WAIT_TIMEOUT, ERR_OVERFLOW = -1, -2, -3, -4, -5


class Tb200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {error_string(code)} (code {code})")
        self.code = code


def _load() -> C.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m thrust_b200.build` "
            "(thrust_b200 has no CPU or PyTorch fallback)")
    lib = C.CDLL(str(_LIB_PATH))
    vp, sz, u64, i32, u32 = C.c_void_p, C.c_size_t, C.c_uint64, C.c_int, C.c_uint32
    psz = C.POINTER(C.c_size_t)
    sigs = {
        "tb200_version": ([], i32),
        "tb200_error_string": ([i32], C.c_char_p),
        "tb200_radix_sort": ([vp, psz, vp, vp, u64, i32, i32, i32, i32, i32, vp], i32),
        "tb200_partition": ([vp, psz, vp, vp, vp, vp, u64, i32, i32, vp, u32, vp, vp], i32),
        "tb200_partition_count": ([vp, psz, vp, u64, i32, i32, vp, u32, vp, vp], i32),
        "tb200_partition_scatter": ([vp, psz, vp, vp, u64, i32, i32, vp, u32, vp, vp, vp], i32),
        "tb200_partition_ties": ([vp, psz, vp, vp, vp, vp, u64, i32, i32, vp, vp, u32, u64, vp, vp], i32),
        "tb200_partition_count_ties": ([vp, psz, vp, u64, i32, i32, vp, vp, u32, u64, vp, vp], i32),
        "tb200_partition_scatter_ties": ([vp, psz, vp, vp, u64, i32, i32, vp, vp, u32, u64, vp, vp, vp], i32),
        "tb200_gather_segments": ([vp, vp, vp, vp, u32, i32, u32, vp, vp], i32),
        "tb200_radix_sort_begin": ([vp, psz, u64, i32, i32, vp], i32),
        "tb200_radix_sort_finish": ([vp, psz, vp, vp, u64, i32, i32, vp], i32),
        "tb200_scan": ([vp, psz, vp, vp, u64, i32, i32, vp, vp], i32),
        "tb200_scan_static": ([vp, vp, u64, i32, i32, vp, vp], i32),
        "tb200_scan_static_status": ([vp], i32),
        "tb200_reduce_by_key": ([vp, psz, vp, vp, vp, vp, vp, u64, i32, i32, vp], i32),
        "tb200_reduce": ([vp, psz, vp, u64, i32, vp, vp, vp], i32),
        "tb200_scan_by_key": ([vp, psz, vp, vp, vp, u64, i32, i32, i32, vp, vp], i32),
        "tb200_unique_by_key": ([vp, psz, vp, vp, vp, vp, vp, u64, i32, i32, vp], i32),
        "tb200_copy_flagged": ([vp, psz, vp, vp, vp, vp, u64, i32, i32, vp], i32),
        "tb200_histogram_sorted": ([vp, u64, i32, vp, u32, vp, vp], i32),
        "tb200_temp_status": ([vp, vp], i32),
        "tb200_selftest_wait_timeout": ([u32, vp], i32),
        "tb200_trace_begin": ([vp], i32),
        "tb200_trace_end": ([C.POINTER(C.c_float), C.POINTER(C.c_int), i32], i32),
        "tb200_workspace_acquire": ([sz, vp, C.POINTER(vp)], i32),
        "tb200_workspace_release": ([vp], i32),
        "tb200_workspace_stats": ([C.POINTER(u64), C.POINTER(u64)], i32),
        "tb200_workspace_release_all": ([], i32),
        "tb200_radix_sort_host": ([vp, vp, u64, i32, i32, i32, vp], i32),
        "tb200_scan_host": ([vp, vp, u64, i32, i32, vp, vp], i32),
        "tb200_reduce_by_key_host": ([vp, vp, vp, vp, C.POINTER(u64), u64, i32, i32, vp], i32),
    }
    for name, (argtypes, restype) in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return lib


lib = _load()

EXPORTS = [
    "tb200_version", "tb200_error_string", "tb200_radix_sort", "tb200_partition", "tb200_partition_count", "tb200_partition_scatter", "tb200_partition_ties", "tb200_partition_count_ties", "tb200_partition_scatter_ties", "tb200_gather_segments", "tb200_radix_sort_begin", "tb200_radix_sort_finish", "tb200_scan", "tb200_scan_static", "tb200_scan_static_status", "tb200_reduce_by_key", "tb200_reduce", "tb200_scan_by_key", "tb200_unique_by_key", "tb200_copy_flagged",
    "tb200_histogram_sorted", "tb200_temp_status", "tb200_selftest_wait_timeout", "tb200_trace_begin", "tb200_trace_end",
    "tb200_workspace_acquire",
    "tb200_workspace_release", "tb200_workspace_stats", "tb200_workspace_release_all", "tb200_radix_sort_host", "tb200_scan_host",
    "tb200_reduce_by_key_host",
]


def error_string(code: int) -> str:
    return lib.tb200_error_string(code).decode()


def check(code: int, what: str) -> None:
    if code != OK:
        raise Tb200Error(code, what)
