"""Host-side logic of the sharded sample sort over gloo, world size 2 and 3, on CPU.

The per-shard compute is injected (a numpy `ops` object backed by the CPU oracle), so these
tests exercise exactly the orchestration the GPU path runs: sampling, splitter choice, the
count exchange, all-to-all-v sizes, source-rank order of the received runs, the capacity
check — and compare the concatenated result with a single-process stable sort.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


class OracleOps:
    """CPU stand-in for DeviceOps: same methods, numpy + the oracle's radix sort."""

    def __init__(self):
        import oracle
        self.chk = oracle.port()

    def sort_pairs(self, keys, vals, n):
        k = keys[:n].numpy().view(np.uint64)
        v = vals[:n].numpy().view(np.uint32)
        self.chk.sort_by_key_inplace(k, v)

    def sort_keys(self, keys):
        self.chk.sort_inplace(keys.numpy().view(np.uint64))

    def segment_counts(self, sorted_keys, n, splitters):
        k = sorted_keys[:n].numpy().view(np.uint64)
        ub = np.searchsorted(k, splitters.numpy().view(np.uint64), side="right")
        return torch.from_numpy(np.diff(np.concatenate([[0], ub])).astype(np.int64))

    def partition(self, keys, vals, n, splitters, out_k, out_v, split_idx=None, index_base=0):
        k = keys[:n].numpy().view(np.uint64)
        sp = splitters.numpy().view(np.uint64)
        if split_idx is None:
            bucket = np.searchsorted(sp, k, side="left")  # number of splitters strictly below the key
        else:  # (key, global index) pairs: number of splitter pairs strictly below the element's pair
            g = np.arange(n, dtype=np.int64) + index_base
            si = split_idx.numpy()
            below = (sp[None, :] < k[:, None]) | ((sp[None, :] == k[:, None]) & (si[None, :] < g[:, None]))
            bucket = below.sum(axis=1)
        order = np.argsort(bucket, kind="stable")
        out_k[:n] = torch.from_numpy(k[order].view(np.int64))
        out_v[:n] = torch.from_numpy(vals[:n].numpy()[order])
        return torch.from_numpy(np.bincount(bucket, minlength=sp.size + 1).astype(np.int64))

    def status(self):
        return 0

    def release(self):
        pass


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, key_bits, slack, out_dir, pipeline="partition_first"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from thrust_b200.sample_sort import ShardedSorter
    rng = np.random.default_rng(1234 + rank)
    keys = rng.integers(0, 1 << key_bits, size=n, dtype=np.uint64) << np.uint64(64 - key_bits)  # spans the sign bit
    vals = (np.arange(n, dtype=np.uint64) + rank * n).astype(np.uint32)
    np.save(f"{out_dir}/in_k{rank}.npy", keys)
    np.save(f"{out_dir}/in_v{rank}.npy", vals)
    sorter = ShardedSorter(n, torch.device("cpu"), world, rank, ops=OracleOps(), slack=slack, pipeline=pipeline)
    k = torch.from_numpy(keys.view(np.int64).copy())
    v = torch.from_numpy(vals.view(np.int32).copy())
    try:
        ok, ov, m = sorter.sort(k, v)
        np.save(f"{out_dir}/out_k{rank}.npy", ok[:m].numpy().view(np.uint64))
        np.save(f"{out_dir}/out_v{rank}.npy", ov[:m].numpy().view(np.uint32))
        send, recv = sorter.last_counts
        assert sum(send) == n and sum(recv) == m
    except OverflowError:
        Path(f"{out_dir}/overflow{rank}").touch()
    dist.barrier()
    dist.destroy_process_group()


def _run(world, n, key_bits, slack, tmp_path, pipeline="partition_first"):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n, key_bits, slack, str(tmp_path), pipeline), nprocs=world, join=True)


@pytest.mark.parametrize("world,n,key_bits,pipeline", [(2, 5000, 64, "partition_first"), (3, 4099, 64, "partition_first"),
                                                       (2, 3000, 6, "partition_first"), (2, 5000, 64, "sort_first"),
                                                       (3, 3000, 6, "sort_first")])
def test_sharded_sort_matches_single_process_stable_sort(tmp_path, world, n, key_bits, pipeline):
    import oracle
    oracle.build(ref=False)
    _run(world, n, key_bits, 1.0 if key_bits < 16 else 1.0 / 4, tmp_path, pipeline)
    in_k = np.concatenate([np.load(tmp_path / f"in_k{r}.npy") for r in range(world)])
    in_v = np.concatenate([np.load(tmp_path / f"in_v{r}.npy") for r in range(world)])
    out_k = np.concatenate([np.load(tmp_path / f"out_k{r}.npy") for r in range(world)])
    out_v = np.concatenate([np.load(tmp_path / f"out_v{r}.npy") for r in range(world)])
    want_k, want_v = oracle.port().sort_by_key(in_k, in_v)
    assert out_k.tobytes() == want_k.tobytes()
    assert out_v.tobytes() == want_v.tobytes()  # stability across ranks: lower source rank first


def test_receive_overflow_is_an_error_not_a_crash(tmp_path):
    # all keys equal and compared by key alone (sort_first): everything goes to one rank, which cannot hold it
    _run(2, 4000, 1, 1.0 / 64, tmp_path, "sort_first")
    assert any((tmp_path / f"overflow{r}").exists() for r in range(2))


@pytest.mark.parametrize("world,key_bits", [(2, 1), (3, 1), (3, 2)])
def test_a_few_heavy_keys_are_divided_between_the_ranks_in_input_order(tmp_path, world, key_bits):
    # one or a few distinct keys: all copies of a key cannot go to one rank; the partition compares
    # (key, global index) pairs, the result is still the single-process stable sort
    import oracle
    oracle.build(ref=False)
    n = 4000
    _run(world, n, key_bits, 1.0 / 8, tmp_path)
    assert not any((tmp_path / f"overflow{r}").exists() for r in range(world))
    in_k = np.concatenate([np.load(tmp_path / f"in_k{r}.npy") for r in range(world)])
    in_v = np.concatenate([np.load(tmp_path / f"in_v{r}.npy") for r in range(world)])
    outs = [np.load(tmp_path / f"out_k{r}.npy") for r in range(world)]
    assert max(o.size for o in outs) <= n + n // 8 + 1024
    out_k = np.concatenate(outs)
    out_v = np.concatenate([np.load(tmp_path / f"out_v{r}.npy") for r in range(world)])
    want_k, want_v = oracle.port().sort_by_key(in_k, in_v)
    assert out_k.tobytes() == want_k.tobytes() and out_v.tobytes() == want_v.tobytes()


def test_sample_positions_and_splitters():
    from thrust_b200.sample_sort import pick_splitters, sample_positions
    p = sample_positions(1 << 20, 1024)
    assert p.numel() == 1024 and p[0] == 512 and p[-1] == (1 << 20) - 512 and bool((p[1:] > p[:-1]).all())
    assert sample_positions(10, 1024).tolist() == list(range(10))
    assert sample_positions(0, 1024).numel() == 0
    s = pick_splitters(torch.arange(4096), 4)
    assert s.tolist() == [1024, 2048, 3072]
    assert pick_splitters(torch.arange(8), 1).numel() == 0


def test_push_offsets_keep_source_rank_order():
    """The push form of the exchange emulated in one process with numpy: every rank scatters its
    buckets into the destinations' receive buffers at push_offsets; the receive buffers must then
    hold the runs in source-rank order, which makes the final stable sort the global stable sort."""
    from thrust_b200.sample_sort import push_offsets
    rng = np.random.default_rng(5)
    world, n = 4, 3001
    shards = [rng.integers(0, 1 << 16, size=n, dtype=np.uint64) for _ in range(world)]
    splitters = np.array([1 << 14, 1 << 15, 3 << 14], dtype=np.uint64)
    buckets = [np.searchsorted(splitters, s, side="left") for s in shards]
    matrix = [[int((b == d).sum()) for d in range(world)] for b in buckets]
    recv = [np.zeros(sum(matrix[r][d] for r in range(world)), dtype=np.uint64) for d in range(world)]
    src = [np.zeros(recv[d].size, dtype=np.int64) for d in range(world)]
    for r in range(world):
        off = push_offsets(matrix, r)
        assert off == [sum(matrix[q][d] for q in range(r)) for d in range(world)]
        for d in range(world):
            run = shards[r][buckets[r] == d]
            recv[d][off[d]:off[d] + run.size] = run
            src[d][off[d]:off[d] + run.size] = r
    whole = np.concatenate(shards)
    order = np.argsort(whole, kind="stable")
    got = np.concatenate([np.sort(recv[d], kind="stable") for d in range(world)])
    assert got.tobytes() == whole[order].tobytes()
    for d in range(world):
        assert (np.diff(src[d]) >= 0).all()  # runs of rank 0, then rank 1, ...
