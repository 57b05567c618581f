"""Helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np
import torch

_NP_TO_TORCH = {
    np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8, np.dtype(np.int16): torch.int16,
    np.dtype(np.uint16): torch.uint16, np.dtype(np.int32): torch.int32, np.dtype(np.uint32): torch.uint32,
    np.dtype(np.int64): torch.int64, np.dtype(np.uint64): torch.uint64, np.dtype(np.float32): torch.float32,
    np.dtype(np.float64): torch.float64, np.dtype(np.bool_): torch.bool,
}


def to_device(a: np.ndarray, device="cuda:0", offset_elems: int = 0) -> torch.Tensor:
    """Copy a numpy array to the GPU bit for bit. offset_elems > 0 places it that many
    elements past an allocation boundary (to exercise pointers that are not 16-byte aligned)."""
    a = np.ascontiguousarray(a)
    raw = torch.from_numpy(a.view(np.uint8).reshape(-1).copy())
    buf = torch.empty(raw.numel() + offset_elems * a.itemsize, dtype=torch.uint8, device=device)
    dst = buf[offset_elems * a.itemsize:]
    dst.copy_(raw)
    return dst.view(_NP_TO_TORCH[a.dtype])


def to_host(t: torch.Tensor, dtype) -> np.ndarray:
    return t.contiguous().view(torch.uint8).cpu().numpy().view(dtype).copy()


def random_keys(rng: np.random.Generator, n: int, dtype, bits=None) -> np.ndarray:
    """Uniform random keys over the whole range of dtype (floats: random bit patterns, so NaNs,
    infinities, subnormals and both zeros occur); `bits` masks keys to their low bits."""
    dt = np.dtype(dtype)
    if dt == np.bool_:
        return rng.integers(0, 2, size=n).astype(np.bool_)
    u = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[dt.itemsize]
    raw = rng.integers(0, np.iinfo(u).max, size=n, dtype=u, endpoint=True)
    if bits is not None:
        raw &= u((1 << bits) - 1) if bits < 8 * dt.itemsize else np.iinfo(u).max
    return raw.view(dt)
