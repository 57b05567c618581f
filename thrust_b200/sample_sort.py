"""Sharded stable sort_by_key across the GPUs of one node: a sample sort.

The reference has no multi-GPU code at all; this is the sharded form of its
``stable_sort_by_key`` on (uint64 key, uint32 value) pairs, one process per GPU.
Two pipelines share the sampling, splitter and exchange code:

``pipeline="partition_first"`` (default; one full local sort per step)
  1. regular sample of the shard: ``samples_per_rank`` keys at evenly spaced positions
  2. all-gather the samples; every rank sorts them identically and takes the keys
     at ranks samples_per_rank * r (r = 1..G-1) as splitters. When one key makes up
     a sixteenth of a rank's share of the sample or more, elements and splitters are
     compared as (key, global index) pairs from here on, so that the copies of one
     key can be divided between ranks, in input order
  3. stable partition of the shard into G buckets, destination d owning the keys in
     (splitter[d-1], splitter[d]] (tb200_partition*: one onesweep pass)
  4. all-gather of the G x G count matrix, then the exchange: the partition pass
     stores every bucket straight into its destination's receive buffer over NVLink
     ("push", the default on GPUs), or all-to-all-v of keys and of values over NCCL;
     received runs are stored in source-rank order
  5. local onesweep sort of the received pairs (tb200_radix_sort). Rank r holds
     global indices [r*n, (r+1)*n), so a stable sort of runs concatenated in
     source-rank order reproduces the single-process stable order.

``pipeline="sort_first"``
  local sort first; the sample is then taken at fixed ranks of the sorted shard
  (a classical regular sample, receive imbalance bounded by n*G/samples), the send
  segments are contiguous ranges found by upper-bound search (tb200_histogram_sorted)
  with no data movement, and step 5 sorts runs that are already sorted. It costs a
  second full local sort and exists for comparison.

``engine="c"`` runs the partition_first pipeline as ONE call of the C entry point
tb200_sample_sort (include/thrust_b200_nccl.h) on a raw NCCL communicator.

The collectives go through ``torch.distributed`` (NCCL on GPUs). The per-shard
compute goes through an ``ops`` object; the default ``DeviceOps`` calls the CUDA
library and there is no CPU implementation in this package (tests inject one to
exercise the orchestration over gloo).
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Optional, Tuple

import torch
import torch.distributed as dist

SAMPLES_PER_RANK = 16384  # the largest share exceeds the mean by ~1.3 % at eight ranks (5 % with 1024): the slowest rank sets the step
CAPACITY_PAD = 1024  # added to every receive capacity: absorbs the rounding of tiny shards


class DeviceOps:
    """Per-shard steps on the GPU through the C ABI."""

    def __init__(self, device: torch.device, capacity: int):
        from . import _capi as capi
        self.capi = capi
        self.device = device
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_radix_sort(None, C.byref(need), None, None, capacity, capi.U64, 4, 0, 0, 64, None),
                   "tb200_radix_sort(size)")
        self.temp = torch.empty(need.value, dtype=torch.uint8, device=device)
        self.small_temp = torch.empty(8 << 20, dtype=torch.uint8, device=device)

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def sort_pairs(self, keys: torch.Tensor, vals: torch.Tensor, n: int) -> None:
        capi = self.capi
        have = C.c_size_t(self.temp.numel())
        capi.check(capi.lib.tb200_radix_sort(C.c_void_p(self.temp.data_ptr()), C.byref(have),
                                             C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()), n, capi.U64, 4,
                                             0, 0, 64, self._stream()), "tb200_radix_sort")

    def sort_keys(self, keys: torch.Tensor) -> None:
        capi = self.capi
        have = C.c_size_t(self.small_temp.numel())
        capi.check(capi.lib.tb200_radix_sort(C.c_void_p(self.small_temp.data_ptr()), C.byref(have),
                                             C.c_void_p(keys.data_ptr()), None, keys.numel(), capi.U64, 0, 0, 0, 64,
                                             self._stream()), "tb200_radix_sort(samples)")

    def segment_counts(self, sorted_keys: torch.Tensor, n: int, splitters: torch.Tensor) -> torch.Tensor:
        """counts[d] = keys in (splitter[d-1], splitter[d]] for d < G-1 (uint64 order), int64 tensor of G-1."""
        capi = self.capi
        counts = torch.empty(splitters.numel(), dtype=torch.int32, device=self.device)
        capi.check(capi.lib.tb200_histogram_sorted(C.c_void_p(sorted_keys.data_ptr()), n, capi.U64,
                                                   C.c_void_p(splitters.data_ptr()), splitters.numel(),
                                                   C.c_void_p(counts.data_ptr()), self._stream()),
                   "tb200_histogram_sorted")
        return counts.to(torch.int64) & 0xFFFFFFFF

    # In the three partition calls ``split_idx`` (int64 tensor or None) turns splitters and elements into
    # (key, index) pairs, element g of the shard having index ``index_base + g``: equal keys can then
    # be divided between buckets, in input order.
    def partition(self, keys: torch.Tensor, vals: torch.Tensor, n: int, splitters: torch.Tensor,
                  out_k: torch.Tensor, out_v: torch.Tensor, split_idx: Optional[torch.Tensor] = None,
                  index_base: int = 0) -> torch.Tensor:
        """Stable partition into len(splitters)+1 buckets; returns the bucket sizes (int64 tensor)."""
        capi = self.capi
        counts = torch.empty(splitters.numel() + 1, dtype=torch.int64, device=self.device)
        have = C.c_size_t(self.temp.numel())
        capi.check(capi.lib.tb200_partition_ties(
            C.c_void_p(self.temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()),
            C.c_void_p(out_k.data_ptr()), C.c_void_p(out_v.data_ptr()), n, capi.U64, 4,
            C.c_void_p(splitters.data_ptr()), C.c_void_p(split_idx.data_ptr()) if split_idx is not None else None,
            splitters.numel(), index_base, C.c_void_p(counts.data_ptr()), self._stream()), "tb200_partition")
        return counts

    def partition_count(self, keys: torch.Tensor, n: int, splitters: torch.Tensor,
                        split_idx: Optional[torch.Tensor] = None, index_base: int = 0) -> torch.Tensor:
        """Bucket sizes of the stable partition by ``splitters`` (int64 tensor); first half of a push."""
        capi = self.capi
        counts = torch.empty(splitters.numel() + 1, dtype=torch.int64, device=self.device)
        have = C.c_size_t(self.temp.numel())
        capi.check(capi.lib.tb200_partition_count_ties(
            C.c_void_p(self.temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), n, capi.U64, 4,
            C.c_void_p(splitters.data_ptr()), C.c_void_p(split_idx.data_ptr()) if split_idx is not None else None,
            splitters.numel(), index_base, C.c_void_p(counts.data_ptr()), self._stream()), "tb200_partition_count")
        return counts

    def partition_scatter(self, keys: torch.Tensor, vals: torch.Tensor, n: int, splitters: torch.Tensor,
                          bucket_keys, bucket_vals, split_idx: Optional[torch.Tensor] = None,
                          index_base: int = 0) -> None:
        """Second half: bucket b goes to the device addresses bucket_keys[b] / bucket_vals[b]
        (integers; peer mappings allowed)."""
        capi = self.capi
        g = splitters.numel() + 1
        pk = (C.c_void_p * g)(*bucket_keys)
        pv = (C.c_void_p * g)(*bucket_vals)
        have = C.c_size_t(self.temp.numel())
        capi.check(capi.lib.tb200_partition_scatter_ties(
            C.c_void_p(self.temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()), n,
            capi.U64, 4, C.c_void_p(splitters.data_ptr()),
            C.c_void_p(split_idx.data_ptr()) if split_idx is not None else None, splitters.numel(), index_base,
            pk, pv, self._stream()), "tb200_partition_scatter")

    def sort_begin(self, n: int) -> None:
        """First half of sort_pairs: clears the scratch; the key gather then counts the digits."""
        capi = self.capi
        have = C.c_size_t(self.temp.numel())
        capi.check(capi.lib.tb200_radix_sort_begin(C.c_void_p(self.temp.data_ptr()), C.byref(have), n, capi.U64, 4,
                                                   self._stream()), "tb200_radix_sort_begin")

    def sort_finish(self, keys: torch.Tensor, vals: torch.Tensor, n: int) -> None:
        capi = self.capi
        have = C.c_size_t(self.temp.numel())
        capi.check(capi.lib.tb200_radix_sort_finish(C.c_void_p(self.temp.data_ptr()), C.byref(have),
                                                    C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()), n,
                                                    capi.U64, 4, self._stream()), "tb200_radix_sort_finish")

    def gather(self, dst: torch.Tensor, src_ptrs, src_offsets, counts, elem_bytes: int, rotate: int = 0,
               count_digits: bool = False) -> None:
        """dst[:sum(counts)] = concatenation of counts[s] elements at src_ptrs[s] + src_offsets[s]
        (device pointers, possibly peer mappings): tb200_gather_segments."""
        capi = self.capi
        g = len(counts)
        ptrs = (C.c_void_p * g)(*src_ptrs)
        offs = (C.c_uint64 * g)(*src_offsets)
        cnts = (C.c_uint64 * g)(*counts)
        hist = C.c_void_p(self.temp.data_ptr()) if count_digits else None
        capi.check(capi.lib.tb200_gather_segments(C.c_void_p(dst.data_ptr()), ptrs, offs, cnts, g, elem_bytes, rotate,
                                                  hist, self._stream()), "tb200_gather_segments")

    def status(self) -> int:
        return int(self.capi.lib.tb200_temp_status(C.c_void_p(self.temp.data_ptr()), self._stream()))

    def release(self) -> None:
        self.temp = None
        self.small_temp = None


def sample_positions(n: int, samples: int) -> torch.Tensor:
    """Ranks of the regular sample inside a sorted shard of n keys (mid-points of equal strides)."""
    s = min(samples, n)
    if s == 0:
        return torch.empty(0, dtype=torch.int64)
    idx = (2 * torch.arange(s, dtype=torch.int64) + 1) * n // (2 * s)
    return idx.clamp_(max=n - 1)


def pick_splitters(sorted_samples: torch.Tensor, world: int) -> torch.Tensor:
    """G-1 splitters: the keys at ranks (len/G)*r of the sorted gathered sample."""
    m = sorted_samples.numel()
    pos = (torch.arange(1, world, dtype=torch.int64) * m) // world
    return sorted_samples[pos.to(sorted_samples.device)]


def push_offsets(matrix, rank: int):
    """matrix[r][b] = pairs rank r sends to rank b. Returns, for every destination b, the element
    offset inside b's receive buffer where THIS rank's bucket starts: the buckets of lower source
    ranks come first, which keeps the received runs in source-rank order."""
    world = len(matrix)
    return [int(sum(matrix[r][b] for r in range(rank))) for b in range(world)]


class ShardedSorter:
    """Sorts one shard per rank; after ``sort`` rank r holds the r-th slice of the global order."""

    def __init__(self, n: int, device: torch.device, world_size: int = 1, rank: int = 0, seed: int = 0,
                 ops=None, group=None, slack: Optional[float] = None, pipeline: str = "partition_first",
                 exchange: str = "auto", engine: str = "python"):
        """engine: "python" — this class runs the steps (torch.distributed collectives around the
        C-ABI kernels); "c" — the whole step is ONE call of tb200_sample_sort
        (include/thrust_b200_nccl.h) on a raw NCCL communicator made for it, and this class only
        owns the buffers (partition_first pipeline, "push" or "nccl" exchange).
        exchange: "push" — the partition kernel stores every bucket straight into its
        destination GPU's receive buffer over NVLink (receive buffers in torch symmetric memory,
        plain peer stores, no multicast), so partition and exchange are one pass over the shard;
        "peer" — partition locally, then every GPU pulls its runs out of the other GPUs' partition
        buffers with one kernel of peer loads; "nccl" — all-to-all-v through torch.distributed;
        "auto" — "push" on CUDA with the partition_first pipeline when the symmetric-memory
        rendezvous succeeds, else "nccl"."""
        if pipeline not in ("partition_first", "sort_first"):
            raise ValueError(pipeline)
        if exchange not in ("auto", "push", "peer", "nccl"):
            raise ValueError(exchange)
        self.n, self.device, self.world, self.rank, self.seed = n, device, world_size, rank, seed
        self.group = group
        self.pipeline = pipeline
        if slack is None:
            # sort_first: a regular sample of sorted shards bounds the imbalance by n*G/samples;
            # partition_first: the sample is random with respect to key order, so the receive
            # count fluctuates by a few percent (about 4 sigma for 8 ranks x 1024 samples)
            slack = 1.0 / 64 if pipeline == "sort_first" else 0.2
        self.capacity = n if world_size == 1 else n + int(n * slack) + CAPACITY_PAD
        if ops is None:
            if device.type != "cuda":
                raise RuntimeError("thrust_b200 has no CPU path: ShardedSorter needs a CUDA device")
            ops = DeviceOps(device, self.capacity)
        self.ops = ops
        self.recv_k = self.recv_v = self.part_k = self.part_v = None
        self.exchange = "none"
        if world_size > 1:
            self.exchange = "nccl"
            self.peer_k = self.peer_v = None
            if pipeline == "partition_first":
                want = exchange if exchange in ("push", "peer") else ("push" if exchange == "auto" and device.type == "cuda" else None)
                if want is not None:
                    try:
                        self._alloc_symmetric(n, want)
                        self.exchange = want
                    except Exception as e:  # symmetric memory unavailable: use the collective
                        if exchange in ("push", "peer"):
                            raise
                        self.exchange_fallback_reason = repr(e)
                if self.exchange == "nccl":
                    self.part_k = torch.empty(n, dtype=torch.int64, device=device)
                    self.part_v = torch.empty(n, dtype=torch.int32, device=device)
            if self.recv_k is None:
                self.recv_k = torch.empty(self.capacity, dtype=torch.int64, device=device)
                self.recv_v = torch.empty(self.capacity, dtype=torch.int32, device=device)
        self.last_counts = None
        self._marks = []
        if engine not in ("python", "c"):
            raise ValueError(engine)
        self.engine = engine if world_size > 1 else "python"
        if self.engine == "c":
            if pipeline != "partition_first" or self.exchange not in ("push", "nccl") or device.type != "cuda":
                raise ValueError("engine='c' runs the partition_first pipeline with the push or nccl exchange on CUDA")
            from . import nccl_sort
            self._nccl_sort = nccl_sort
            self._comm = nccl_sort.create_comm(rank, world_size, device, group)
            push = self.exchange == "push"
            self.part_k = self.part_v = None  # the C entry keeps its partition buffers in its scratch
            self._c_temp = torch.empty(nccl_sort.temp_bytes(world_size, n, self.capacity, push), dtype=torch.uint8,
                                       device=device)

    def _alloc_symmetric(self, n: int, mode: str) -> None:
        """Buffers the peers touch, in symmetric memory, and every rank's pointers to them:
        the partition buffers for "peer" (pulled from), the receive buffers for "push"."""
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads and stores only
        import torch.distributed._symmetric_memory as symm
        grp = self.group if self.group is not None else dist.group.WORLD
        size = n if mode == "peer" else self.capacity
        buf_k = symm.empty(size, dtype=torch.int64, device=self.device)
        buf_v = symm.empty(size, dtype=torch.int32, device=self.device)
        hk = symm.rendezvous(buf_k, grp)
        hv = symm.rendezvous(buf_v, grp)
        self.peer_k = [int(p) for p in hk.buffer_ptrs]
        self.peer_v = [int(p) for p in hv.buffer_ptrs]
        self._symm_handles = (hk, hv)
        if len(self.peer_k) != self.world:
            raise RuntimeError("symmetric memory rendezvous returned the wrong number of peers")
        if mode == "peer":
            self.part_k, self.part_v = buf_k, buf_v
        else:
            self.recv_k, self.recv_v = buf_k, buf_v

    def _mark(self, name: str) -> None:
        """Records a CUDA event at a phase boundary (device tensors only)."""
        if self.device.type == "cuda":
            e = torch.cuda.Event(enable_timing=True)
            e.record(torch.cuda.current_stream(self.device))
            self._marks.append((name, e))

    def phase_times(self) -> dict:
        """Milliseconds between the phase boundaries of the last sort() (synchronises)."""
        if len(self._marks) < 2:
            return {}
        self._marks[-1][1].synchronize()
        return {self._marks[i + 1][0]: self._marks[i][1].elapsed_time(self._marks[i + 1][1])
                for i in range(len(self._marks) - 1)}

    def release(self) -> None:
        self.ops.release()
        self.recv_k = self.recv_v = self.part_k = self.part_v = None

    def check_status(self) -> None:
        st = self.ops.status()
        if st != 0:
            raise RuntimeError(f"device status {st} after sharded sort")

    def sort(self, keys: torch.Tensor, vals: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """keys: int64 tensor holding uint64 bit patterns, vals: int32 tensor holding uint32.
        Returns (keys, vals, count): this rank's slice of the globally sorted sequence."""
        n, G = self.n, self.world
        if G == 1:
            self.ops.sort_pairs(keys, vals, n)
            return keys, vals, n
        sort_first = self.pipeline == "sort_first"
        self._marks = []
        self._mark("start")
        if self.engine == "c":
            push = self.exchange == "push"
            m = self._nccl_sort.sample_sort(self._comm, self.rank, G, keys[:n], vals[:n], self.recv_k, self.recv_v,
                                            self.peer_k if push else None, self.peer_v if push else None,
                                            self._c_temp)
            self.last_counts = None
            self._mark("sample_sort_c")
            return self.recv_k, self.recv_v, m
        if sort_first:
            self.ops.sort_pairs(keys, vals, n)
            self._mark("local_sort")
        # regular sample -> splitters (identical on every rank)
        pos = sample_positions(n, SAMPLES_PER_RANK).to(self.device)
        mine = keys[pos].contiguous()
        gathered = torch.empty(G * mine.numel(), dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(gathered, mine, group=self.group)
        split_idx, index_base = None, self.rank * n
        if sort_first:
            self.ops.sort_keys(gathered)
        else:
            # The sample also tells whether a few keys make up so much of the input that all copies of one
            # key cannot go to one rank. Then elements are compared as (key, global index) pairs, and so
            # are the splitters: the sample is sorted with each key's ordinal as its value (a stable sort
            # of a rank-major, position-ascending sample leaves equal keys in index order).
            ordinal = torch.arange(gathered.numel(), dtype=torch.int32, device=self.device)
            self.ops.sort_pairs(gathered, ordinal, gathered.numel())
            heaviest = int(torch.unique_consecutive(gathered, return_counts=True)[1].max())
            if heaviest * 16 >= mine.numel():  # one key holds a sixteenth of a rank's share or more
                where = ordinal.long()
                sample_index = (where // mine.numel()) * n + pos[where % mine.numel()]
                split_idx = pick_splitters(sample_index, G).contiguous()
        splitters = pick_splitters(gathered, G).contiguous()
        self.split_ties = split_idx is not None
        self._mark("sample_and_splitters")
        if sort_first:
            # contiguous send segments of the sorted shard
            head = self.ops.segment_counts(keys, n, splitters)
            send = torch.cat([head, (n - head.sum()).reshape(1)])
            src_k, src_v = keys, vals
        elif self.exchange == "push":
            send = self.ops.partition_count(keys, n, splitters, split_idx, index_base)
            src_k = src_v = None
        else:
            send = self.ops.partition(keys, vals, n, splitters, self.part_k, self.part_v, split_idx, index_base)
            src_k, src_v = self.part_k, self.part_v
        self._mark("segments" if sort_first else ("bucket_counts" if self.exchange == "push" else "partition"))
        # 5. the whole G x G count matrix goes to every rank (row r = what rank r sends), so all
        # ranks take the same decision about receive overflow; then the payload
        matrix = torch.empty(G * G, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(matrix, send.contiguous(), group=self.group)
        mat = matrix.cpu().view(G, G)
        send_l = mat[self.rank].tolist()
        recv_l = mat[:, self.rank].tolist()
        m = int(sum(recv_l))
        self.last_counts = (send_l, recv_l)
        worst = int(mat.sum(dim=0).max())
        if worst > self.capacity:
            raise OverflowError(f"{worst} incoming pairs on one rank exceed the receive capacity {self.capacity}")
        self._mark("count_matrix")
        if self.exchange == "push" and not sort_first:
            # Push: my bucket for rank b lands in b's receive buffer behind the buckets of lower
            # source ranks. The count matrix arrived through a collective that every rank entered
            # after the previous step's work on its stream, so the receive buffers are free.
            off = push_offsets(mat.tolist(), self.rank)
            self.ops.partition_scatter(keys, vals, n, splitters,
                                       [self.peer_k[b] + 8 * off[b] for b in range(G)],
                                       [self.peer_v[b] + 4 * off[b] for b in range(G)], split_idx, index_base)
            # every rank's stores have landed once every rank's partition kernel has finished
            dist.barrier(group=self.group)
            self._mark("partition_and_exchange")
            self.ops.sort_pairs(self.recv_k, self.recv_v, m)
            self._mark("final_sort")
            return self.recv_k, self.recv_v, m
        if self.exchange == "peer" and not sort_first:
            # Pull: rank r's bucket for me starts where the buckets of lower destinations end.
            # The count matrix arrived through a collective that every rank entered after its
            # partition kernel, so all partition buffers are complete.
            src_off = [int(mat[r, :self.rank].sum()) for r in range(G)]
            # The key gather also counts the digits of all eight passes of the sort that follows.
            self.ops.sort_begin(m)
            self.ops.gather(self.recv_k, self.peer_k, src_off, recv_l, 8, self.rank, count_digits=True)
            self.ops.gather(self.recv_v, self.peer_v, src_off, recv_l, 4, self.rank)
            # nobody may overwrite its partition buffer (next call) before all pulls are done
            dist.barrier(group=self.group)
            self._mark("exchange")
            self.ops.sort_finish(self.recv_k, self.recv_v, m)
            self._mark("final_sort")
            return self.recv_k, self.recv_v, m
        else:
            dist.all_to_all_single(self.recv_k[:m], src_k[:n], recv_l, send_l, group=self.group)
            dist.all_to_all_single(self.recv_v[:m], src_v[:n], recv_l, send_l, group=self.group)
        self._mark("exchange")
        # stable sort of the runs (already in source-rank order)
        self.ops.sort_pairs(self.recv_k, self.recv_v, m)
        self._mark("final_sort")
        return self.recv_k, self.recv_v, m

    # ---- reference-free verification (needs the CUDA library) ------------------------------
    def verify(self, out_k: torch.Tensor, out_v: torch.Tensor, m: int) -> bool:
        """True when the distributed output is the stable sort of keys hash(seed, g), g in [0, G*n)."""
        from . import datagen
        total = self.n * self.world
        res = datagen.check_hashed_pairs(out_k, out_v, m, self.seed, total)
        edge = torch.zeros(4, dtype=torch.int64, device=self.device)  # first key, first value, last key, last value
        if m > 0:
            edge[0], edge[1] = out_k[0], out_v[0].to(torch.int64) & 0xFFFFFFFF
            edge[2], edge[3] = out_k[m - 1], out_v[m - 1].to(torch.int64) & 0xFFFFFFFF
        ok = True
        if self.world > 1:
            dist.all_reduce(res, group=self.group)
            edges = torch.empty(4 * self.world, dtype=torch.int64, device=self.device)
            dist.all_gather_into_tensor(edges, edge, group=self.group)
            e = edges.cpu().view(self.world, 4).tolist()
            for r in range(self.world - 1):
                lo = e[r][2] & 0xFFFFFFFFFFFFFFFF
                hi = e[r + 1][0] & 0xFFFFFFFFFFFFFFFF
                ok = ok and lo <= hi
        r4 = [x & 0xFFFFFFFFFFFFFFFF for x in res.cpu().tolist()]
        want_sum = (total * (total - 1) // 2) & 0xFFFFFFFFFFFFFFFF
        return ok and r4[0] == 0 and r4[1] == 0 and r4[2] == want_sum and r4[3] == total


class _NoOps:
    """Stand-in for the per-shard device steps where only ShardedSorter.verify is wanted."""

    def release(self) -> None:
        pass

    def status(self) -> int:
        return 0


def bench_host_path(n: int, device: torch.device, world: int, rank: int, seed: int, steps: int = 3,
                    warmup: int = 1) -> Optional[dict]:
    """End-to-end timing with HOST buffers: pinned host -> device, sort, device -> pinned host, all inside
    the timed region. One GPU: the C entry point tb200_radix_sort_host. Several GPUs: copies around
    ShardedSorter.sort. Returns the ``e2e`` object of the benchmark line (None if host memory is short)."""
    from . import _capi as capi, datagen as g
    try:
        hk = torch.empty(n, dtype=torch.int64).pin_memory()
        hv = torch.empty(n, dtype=torch.int32).pin_memory()
        if world > 1:
            cap = n + n // 5 + CAPACITY_PAD
            ok_, ov_ = torch.empty(cap, dtype=torch.int64).pin_memory(), torch.empty(cap, dtype=torch.int32).pin_memory()
    except RuntimeError:
        return None
    stream = torch.cuda.current_stream(device)
    st = C.c_void_p(stream.cuda_stream)
    sorter = dk = dv = None
    if world > 1:
        sorter = ShardedSorter(n, device, world, rank, seed)
        dk = torch.empty(n, dtype=torch.int64, device=device)
        dv = torch.empty(n, dtype=torch.int32, device=device)
    times, d2h = [], 0
    for i in range(warmup + steps):
        g.host(g.BITS_U64, n, seed, rank * n, out=hk.numpy().view("uint64"))
        g.host(g.INDEX_U32, n, seed, rank * n, out=hv.numpy().view("uint32"))
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        if world == 1:
            capi.check(capi.lib.tb200_radix_sort_host(C.c_void_p(hk.data_ptr()), C.c_void_p(hv.data_ptr()), n,
                                                      capi.U64, 4, 0, st), "tb200_radix_sort_host")
            d2h = n * 12
        else:
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            rk, rv, m = sorter.sort(dk, dv)
            ok_[:m].copy_(rk[:m], non_blocking=True)
            ov_[:m].copy_(rv[:m], non_blocking=True)
            d2h = m * 12
        b.record(stream)
        b.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
    t = torch.tensor(times, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.mean().item())
    # the last step's result, checked in full: keys AND values must be the stable sort of the hashed
    # pairs (reference-free checker on the device; at one GPU the host result is copied back for it)
    if world == 1:
        capi.lib.tb200_workspace_release_all()
        checker = ShardedSorter(n, device, 1, 0, seed, ops=_NoOps())
        verified = checker.verify(hk.to(device), hv.to(device), n)
    else:
        verified = sorter.verify(rk, rv, m)
        sorter.release()
    return {"value": n * world / (ms * 1e-3) / 1e9, "unit": "Gkeys/s", "h2d_bytes_per_step": n * 12,
            "d2h_bytes_per_step": d2h, "ms_per_step": ms, "steps": steps, "host_memory": "pinned",
            "api": "tb200_radix_sort_host" if world == 1 else "ShardedSorter.sort between pinned-host copies",
            "verified": bool(verified)}
