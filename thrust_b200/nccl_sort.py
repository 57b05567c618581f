"""ctypes binding of tb200_sample_sort (include/thrust_b200_nccl.h, libthrust_b200_nccl.so): the
sharded sort behind one C call, driven with a raw ncclComm_t.

PyTorch does not hand out the communicators of its process groups, so `create_comm` makes one:
rank 0 draws an ncclUniqueId, the id travels through torch.distributed, every rank calls
ncclCommInitRank. The NCCL used is the one already in the process (PyTorch's), which the
library resolves to as well: import torch before this module.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import _capi as capi

_LIB_PATH = Path(__file__).resolve().parent / "libthrust_b200_nccl.so"
ERR_NCCL = -6


class _UniqueId(C.Structure):
    _fields_ = [("internal", C.c_byte * 128)]


def _load():
    if not _LIB_PATH.exists():
        raise ImportError(f"{_LIB_PATH} is missing: run `python -m thrust_b200.build`")
    nccl = C.CDLL("libnccl.so.2", mode=C.RTLD_GLOBAL)  # the copy PyTorch loaded, if any
    lib = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    lib.tb200_sample_sort.restype = C.c_int
    lib.tb200_sample_sort.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_size_t), C.c_void_p,
                                      C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p,
                                      C.c_void_p, C.POINTER(C.c_uint64), C.c_void_p]
    nccl.ncclGetUniqueId.argtypes = [C.POINTER(_UniqueId)]
    nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, _UniqueId, C.c_int]
    nccl.ncclCommDestroy.argtypes = [C.c_void_p]
    return nccl, lib


nccl, lib = _load()


def create_comm(rank: int, world: int, device: torch.device, group=None) -> C.c_void_p:
    """A new NCCL communicator over the ranks of `group` (collective; the current device is used)."""
    uid = _UniqueId()
    if rank == 0 and nccl.ncclGetUniqueId(C.byref(uid)) != 0:
        raise RuntimeError("ncclGetUniqueId failed")
    box = [bytes(uid.internal)]
    dist.broadcast_object_list(box, src=0, group=group, device=device if device.type == "cuda" else None)
    C.memmove(C.byref(uid), box[0], 128)
    comm = C.c_void_p()
    with torch.cuda.device(device):
        if nccl.ncclCommInitRank(C.byref(comm), world, uid, rank) != 0:
            raise RuntimeError("ncclCommInitRank failed")
    return comm


def destroy_comm(comm: C.c_void_p) -> None:
    nccl.ncclCommDestroy(comm)


def temp_bytes(world: int, n: int, capacity: int, push: bool) -> int:
    need = C.c_size_t(0)
    peers = (C.c_void_p * world)() if push else None
    capi.check(lib.tb200_sample_sort(None, 0, world, None, C.byref(need), None, None, n, None, None, capacity,
                                     peers, peers, None, None), "tb200_sample_sort(size)")
    return need.value


def sample_sort(comm, rank: int, world: int, keys: torch.Tensor, vals: torch.Tensor, out_keys: torch.Tensor,
                out_vals: torch.Tensor, peer_keys: Optional[Sequence[int]] = None,
                peer_vals: Optional[Sequence[int]] = None, temp: Optional[torch.Tensor] = None) -> int:
    """keys: int64 tensor of uint64 bit patterns, vals: 4-byte elements; out_* have room for the
    receive capacity. peer_*: every rank's out_* as mapped here (push exchange) or None (NCCL
    send / receive). Returns this rank's count; raises OverflowError on every rank together."""
    n, capacity = keys.numel(), out_keys.numel()
    push = peer_keys is not None
    need = temp_bytes(world, n, capacity, push)
    if temp is None or temp.numel() < need:
        temp = torch.empty(need, dtype=torch.uint8, device=keys.device)
    have = C.c_size_t(temp.numel())
    count = C.c_uint64(0)
    pk = (C.c_void_p * world)(*peer_keys) if push else None
    pv = (C.c_void_p * world)(*peer_vals) if push else None
    with torch.cuda.device(keys.device):
        stream = C.c_void_p(torch.cuda.current_stream(keys.device).cuda_stream)
        rc = lib.tb200_sample_sort(comm, rank, world, C.c_void_p(temp.data_ptr()), C.byref(have),
                                   C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()), n,
                                   C.c_void_p(out_keys.data_ptr()), C.c_void_p(out_vals.data_ptr()), capacity, pk, pv,
                                   C.byref(count), stream)
    if rc == capi.ERR_OVERFLOW:
        raise OverflowError("some rank would receive more pairs than the receive capacity")
    if rc == ERR_NCCL:
        raise RuntimeError("tb200_sample_sort: an NCCL call failed")
    capi.check(rc, "tb200_sample_sort")
    return int(count.value)
