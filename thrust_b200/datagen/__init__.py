"""Seeded synthetic inputs of the benchmark configurations (counter-based, so the
host, the device and every rank produce the same element i for a given seed).

Python front end of ``tb200_datagen`` (datagen.h, built into libtb200_datagen.so next to
this file: test and benchmark support, separate from the algorithm library, which this module
does not load). Device variants return CUDA tensors, host variants fill numpy arrays (or pinned
tensors).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional, Tuple

import numpy as np
import torch

_LIB_PATH = Path(__file__).resolve().parent / "libtb200_datagen.so"
if not _LIB_PATH.exists():
    raise ImportError(f"{_LIB_PATH} is missing: build it with `python -m thrust_b200.build`")


class _Check:
    @staticmethod
    def check(code: int, what: str) -> None:
        if code != 0:
            raise RuntimeError(f"{what} failed with code {code}")


capi = _Check

BITS_U32, BITS_U64, INDEX_U32, UNIFORM_F32, UNIFORM_I64, HEAD_FLAGS_I32, AND3_F32, ZIPF_RANK_U32 = range(8)

_lib = C.CDLL(str(_LIB_PATH))
_lib.tb200_datagen.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_uint64, C.c_void_p,
                               C.c_uint32, C.c_int, C.c_void_p]
_lib.tb200_datagen.restype = C.c_int
_lib.tb200_datagen_hash.argtypes = [C.c_uint64, C.c_uint64]
_lib.tb200_datagen_hash.restype = C.c_uint64
_lib.tb200_check_hashed_pairs.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p,
                                          C.c_void_p]
_lib.tb200_check_hashed_pairs.restype = C.c_int

# seeds of the benchmark configurations
SEED_SORT_I32 = 1337
SEED_SCAN = 7
SEED_RBK = 11
SEED_PAIRS_U64 = 42
SEED_LOW_ENTROPY = 4
SEED_SHARDED = 2024

_KIND_DTYPE = {
    BITS_U32: (torch.int32, np.uint32), BITS_U64: (torch.int64, np.uint64), INDEX_U32: (torch.int32, np.uint32),
    UNIFORM_F32: (torch.float32, np.float32), UNIFORM_I64: (torch.int64, np.int64),
    HEAD_FLAGS_I32: (torch.int32, np.int32), AND3_F32: (torch.float32, np.float32),
    ZIPF_RANK_U32: (torch.int32, np.uint32),
}


def hash64(seed: int, i: int) -> int:
    return int(_lib.tb200_datagen_hash(seed, i))


def check_hashed_pairs(keys: torch.Tensor, vals: torch.Tensor, m: int, seed: int, total: int) -> torch.Tensor:
    """Runs the reference-free checker over the first m (key, value) pairs of one sorted shard; returns
    the 4 x int64 device tensor documented in datagen.h (violations, bad keys, index sum, count)."""
    res = torch.zeros(4, dtype=torch.int64, device=keys.device)
    with torch.cuda.device(keys.device):
        stream = C.c_void_p(torch.cuda.current_stream(keys.device).cuda_stream)
        capi.check(_lib.tb200_check_hashed_pairs(C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()), m, seed, total,
                                                 C.c_void_p(res.data_ptr()), stream), "tb200_check_hashed_pairs")
    return res


def _aux(kind: int, lo=None, hi=None, period=None):
    if kind == UNIFORM_F32:
        return (C.c_float * 2)(lo, hi)
    if kind == UNIFORM_I64:
        return (C.c_int64 * 2)(lo, hi)
    if kind == HEAD_FLAGS_I32:
        return (C.c_uint32 * 1)(period)
    return None


def device(kind: int, n: int, seed: int, first: int = 0, dev="cuda:0", torch_dtype=None, out=None, cdf=None,
           **aux) -> torch.Tensor:
    """Elements first..first+n-1 of stream (kind, seed) as a CUDA tensor."""
    t = out if out is not None else torch.empty(n, dtype=torch_dtype or _KIND_DTYPE[kind][0], device=dev)
    with torch.cuda.device(t.device):
        stream = C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
        if kind == ZIPF_RANK_U32:
            a, alen = C.c_void_p(cdf.data_ptr()), cdf.numel()
        else:
            buf = _aux(kind, **aux)
            a, alen = (C.cast(buf, C.c_void_p) if buf is not None else None), 0
        capi.check(_lib.tb200_datagen(C.c_void_p(t.data_ptr()), n, first, kind, seed, a, alen, 1, stream),
                   "tb200_datagen")
    return t


def host(kind: int, n: int, seed: int, first: int = 0, out: Optional[np.ndarray] = None, cdf=None, **aux) -> np.ndarray:
    """Same stream on the host (numpy array; filled with all host threads)."""
    a = out if out is not None else np.empty(n, dtype=_KIND_DTYPE[kind][1])
    if kind == ZIPF_RANK_U32:
        p, alen = C.c_void_p(cdf.ctypes.data), cdf.size
    else:
        buf = _aux(kind, **aux)
        p, alen = (C.cast(buf, C.c_void_p) if buf is not None else None), 0
    capi.check(_lib.tb200_datagen(C.c_void_p(a.ctypes.data), n, first, kind, seed, p, alen, 0, None), "tb200_datagen")
    return a


def zipf_cdf(num_values: int = 1 << 16, s: float = 1.2) -> np.ndarray:
    w = 1.0 / np.power(np.arange(1, num_values + 1, dtype=np.float64), s)
    c = np.cumsum(w)
    c /= c[-1]
    c[-1] = 1.0
    return c


def zipf_values(num_values: int = 1 << 16) -> np.ndarray:
    """The distinct float32 key values of the Zipf workload, ascending (rank r -> 0.5*r - 1000)."""
    return (0.5 * np.arange(num_values, dtype=np.float64) - 1000.0).astype(np.float32)


# ---- the benchmark configurations (device side) --------------------------------------

def sort_i32(n: int = 1 << 25, dev="cuda:0") -> torch.Tensor:
    """int32 keys uniform over [INT32_MIN, INT32_MAX], seed 1337."""
    return device(BITS_U32, n, SEED_SORT_I32, dev=dev)


def scan_f32(n: int = 1 << 30, dev="cuda:0") -> torch.Tensor:
    return device(UNIFORM_F32, n, SEED_SCAN, dev=dev, lo=-1.0, hi=1.0)


def scan_i64(n: int = 1 << 30, dev="cuda:0") -> torch.Tensor:
    return device(UNIFORM_I64, n, SEED_SCAN, dev=dev, lo=-(1 << 20), hi=1 << 20)


def rbk_inputs(n: int = 1 << 28, dev="cuda:0") -> Tuple[torch.Tensor, torch.Tensor]:
    """Already-grouped int32 keys (run id; run lengths geometric with mean 16) and float32 values
    uniform(-50, 50), seed 11. The run ids are the inclusive scan of the head flags minus one."""
    flags = device(HEAD_FLAGS_I32, n, SEED_RBK, dev=dev, period=16)
    keys = _cumsum_chunks(flags)
    keys.sub_(1)
    vals = device(UNIFORM_F32, n, SEED_RBK + 1, dev=dev, lo=-50.0, hi=50.0)
    return keys, vals


def pairs_u64_u32(n: int, seed: int = SEED_PAIRS_U64, first: int = 0, dev="cuda:0") -> Tuple[torch.Tensor, torch.Tensor]:
    """uint64 keys uniform over 64 bits (stored in int64 tensors) with uint32 value = global index."""
    return device(BITS_U64, n, seed, first, dev=dev), device(INDEX_U32, n, seed, first, dev=dev)


def and3_pairs(n: int = 1 << 28, dev="cuda:0") -> Tuple[torch.Tensor, torch.Tensor]:
    """float32 keys = AND of three random words (low entropy, no NaN), int32 payload = index."""
    return device(AND3_F32, n, SEED_LOW_ENTROPY, dev=dev), device(INDEX_U32, n, 0, dev=dev)


def zipf_pairs(n: int = 1 << 28, dev="cuda:0") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """float32 keys drawn Zipf(1.2) over 65536 distinct values, int32 payload = index; also returns
    the ascending table of the distinct values (the histogram's bin values)."""
    cdf = torch.from_numpy(zipf_cdf()).to(dev)
    table = torch.from_numpy(zipf_values()).to(dev)
    ranks = device(ZIPF_RANK_U32, n, SEED_LOW_ENTROPY + 1, dev=dev, cdf=cdf)
    keys = table[ranks.long()] if n <= (1 << 26) else _gather_chunks(table, ranks)
    return keys, device(INDEX_U32, n, 0, dev=dev), table


def _cumsum_chunks(flags: torch.Tensor, chunk: int = 1 << 26) -> torch.Tensor:
    """In-place inclusive prefix sum of int32 flags with torch (input preparation, not the product path)."""
    carry = 0
    for s in range(0, flags.numel(), chunk):
        part = flags[s:s + chunk]
        part.cumsum_(0)
        if carry:
            part.add_(carry)
        carry = int(part[-1].item()) if part.numel() else carry
    return flags


def _gather_chunks(table: torch.Tensor, ranks: torch.Tensor, chunk: int = 1 << 26) -> torch.Tensor:
    out = torch.empty(ranks.numel(), dtype=table.dtype, device=ranks.device)
    for s in range(0, ranks.numel(), chunk):
        out[s:s + chunk] = table[ranks[s:s + chunk].long()]
    return out
