"""Scan and reduce_by_key over an array that is sharded across GPUs, one process per GPU.

Rank r holds elements [offset_r, offset_r + n_r) of the global array, in rank order. Both
algorithms run the single-GPU kernels on the shard and exchange one small record per rank
(the "block totals" of a scan whose blocks are the shards):

* scan: every rank reduces its shard (one read), the totals are all-gathered, and the shard is
  scanned with the sum of the shards in front as its seed (one read + one write). Three touches
  per element instead of two: there is no way to hide the dependency of shard r on the total of
  shard r - 1 inside one pass without serialising the ranks.
* reduce_by_key: every rank reduces its shard by key; a run that crosses a shard boundary belongs
  to the rank where it starts, and the ranks behind it hand it the sums of their leading runs
  (first key, first sum, last key, run count per rank are all-gathered; every rank decides alone).

The per-shard compute is an `ops` object (`ScanOps`: the C-ABI kernels on CUDA tensors), so the
host logic can be run on CPU ranks over gloo with a stand-in.

The reference has no multi-GPU code; the single-GPU semantics are those of thrust::inclusive_scan /
exclusive_scan (thrust/scan.h:99-284) and thrust::reduce_by_key (thrust/reduce.h:560-620) applied to
the concatenation of the shards.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

_NP = {torch.int32: np.int32, torch.int64: np.int64, torch.float32: np.float32, torch.float64: np.float64}


class ScanOps:
    """The shard-local kernels (CUDA tensors, through the C ABI)."""

    def reduce(self, x: torch.Tensor):
        from . import algorithms as tb
        return tb.reduce(x) if x.numel() else 0

    def scan(self, x: torch.Tensor, out: torch.Tensor, exclusive: bool, seed) -> None:
        from . import algorithms as tb
        if exclusive:
            tb.exclusive_scan(x, out=out, init=seed)
        else:
            tb.inclusive_scan(x, out=out, init=seed)

    def reduce_by_key(self, keys: torch.Tensor, vals: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
        from . import algorithms as tb
        return tb.reduce_by_key(keys, vals)


def _add(dtype, a, b):
    """a + b in the element type (integers wrap like the kernels' arithmetic)."""
    t = _NP[dtype]
    with np.errstate(over="ignore"):
        return t(t(a) + t(b)).item() if np.issubdtype(t, np.integer) else float(t(t(a) + t(b)))


class ShardedScan:
    def __init__(self, world_size: int = 1, rank: int = 0, group=None, ops=None):
        self.world, self.rank, self.group = world_size, rank, group
        self.ops = ops if ops is not None else ScanOps()

    def _gather(self, record):
        if self.world == 1:
            return [record]
        out = [None] * self.world
        dist.all_gather_object(out, record, group=self.group)
        return out

    # ---- scan -------------------------------------------------------------------------------
    def _scan(self, x: torch.Tensor, out: Optional[torch.Tensor], exclusive: bool, init) -> torch.Tensor:
        if x.dtype not in _NP:
            raise TypeError("sharded scan supports int32, int64, float32 and float64")
        if out is None:
            out = torch.empty_like(x)
        totals = self._gather(self.ops.reduce(x))
        seed = 0 if init is None else init
        for r in range(self.rank):  # in rank order: the same grouping on every run
            seed = _add(x.dtype, seed, totals[r])
        if x.numel():
            self.ops.scan(x, out, exclusive, seed)
        return out

    def inclusive_scan(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self._scan(x, out, False, None)

    def exclusive_scan(self, x: torch.Tensor, init=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self._scan(x, out, True, init)

    # ---- reduce_by_key ----------------------------------------------------------------------
    def reduce_by_key(self, keys: torch.Tensor, vals: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """Returns this rank's part of the result: the runs that START in its shard, in order."""
        if vals.dtype not in _NP:
            raise TypeError("sharded reduce_by_key supports int32, int64, float32 and float64 values")
        if keys.numel():
            ko, vo, m = self.ops.reduce_by_key(keys, vals)
            rec = (m, ko[0].item(), vo[0].item(), ko[m - 1].item(), m == 1)
        else:
            ko, vo, m = keys[:0].clone(), vals[:0].clone(), 0
            rec = (0, None, None, None, False)
        recs = self._gather(rec)
        if m == 0:
            return ko, vo, 0
        # does my first run continue a run that started on a rank in front of me?
        drop = 0
        for p in range(self.rank - 1, -1, -1):
            if recs[p][0] == 0:
                continue
            drop = int(recs[p][3] == rec[1])
            break
        # the leading runs of the ranks behind me that continue my last run
        if drop and m == 1:
            return ko[:0], vo[:0], 0  # the whole shard is the middle of somebody else's run
        last, grown = vo[m - 1].item(), False
        for q in range(self.rank + 1, self.world):
            mq, first_key, first_sum, _, single = recs[q]
            if mq == 0:
                continue
            if first_key != rec[3]:
                break
            last, grown = _add(vals.dtype, last, first_sum), True  # left to right, like one sequential pass
            if not single:
                break
        if grown:
            vo[m - 1] = last
        return ko[drop:m], vo[drop:m], m - drop
