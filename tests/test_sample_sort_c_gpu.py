"""The C entry point of the sharded sort, tb200_sample_sort (include/thrust_b200_nccl.h).

One rank: on any GPU box (no communicator needed). Two ranks: spawned as one process per GPU
over NCCL when the box has two GPUs; both exchange forms (ncclSend / ncclRecv, and the partition
pass storing straight into the peers' output buffers) are compared with the single-process
stable sort of the concatenated shards, and an input that cannot fit raises on every rank.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu


def test_one_rank_is_a_stable_local_sort(cuda_device):
    import oracle
    from thrust_b200 import nccl_sort
    from util import to_device, to_host
    rng = np.random.default_rng(3)
    n = 200_003
    keys = rng.integers(0, 1 << 12, size=n, dtype=np.uint64) << np.uint64(52)
    vals = np.arange(n, dtype=np.uint32)
    dk, dv = to_device(keys), to_device(vals)
    ok, ov = torch.empty_like(dk), torch.empty_like(dv)
    m = nccl_sort.sample_sort(None, 0, 1, dk, dv, ok, ov)
    wk, wv = oracle.port().sort_by_key(keys, vals)
    assert m == n
    assert to_host(ok, np.uint64).tobytes() == wk.tobytes() and to_host(ov, np.uint32).tobytes() == wv.tobytes()
    assert to_host(dk, np.uint64).tobytes() == keys.tobytes()  # the input is left alone


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from thrust_b200.sample_sort import ShardedSorter
    n = 300_000 + 17
    rng = np.random.default_rng(99 + rank)
    for case, bits in (("wide", 64), ("narrow", 10), ("heavy", 1)):  # heavy: two keys, divided between the ranks
        keys = rng.integers(0, 1 << bits, size=n, dtype=np.uint64) << np.uint64(64 - bits)
        vals = (np.arange(n, dtype=np.uint64) + rank * n).astype(np.uint32)
        np.save(f"{out_dir}/{case}_in_k{rank}.npy", keys)
        np.save(f"{out_dir}/{case}_in_v{rank}.npy", vals)
        k = torch.from_numpy(keys.view(np.int64)).to(dev)
        v = torch.from_numpy(vals.view(np.int32)).to(dev)
        for exchange in ("nccl", "push"):
            sorter = ShardedSorter(n, dev, world, rank, exchange=exchange, engine="c", slack=0.25)
            ok, ov, m = sorter.sort(k, v)
            if case == "heavy":  # the Python orchestration takes the same decisions
                ok2, ov2, m2 = ShardedSorter(n, dev, world, rank, exchange=exchange, slack=0.25).sort(k, v)
                torch.cuda.synchronize()
                assert m2 == m and torch.equal(ok2[:m], ok[:m]) and torch.equal(ov2[:m], ov[:m])
            torch.cuda.synchronize()
            np.save(f"{out_dir}/{case}_{exchange}_k{rank}.npy", ok[:m].cpu().numpy().view(np.uint64))
            np.save(f"{out_dir}/{case}_{exchange}_v{rank}.npy", ov[:m].cpu().numpy().view(np.uint32))
            dist.barrier()
    # receive buffers smaller than a rank's share: no room, and every rank says so
    k = torch.zeros(n, dtype=torch.int64, device=dev)
    sorter = ShardedSorter(n, dev, world, rank, exchange="nccl", engine="c", slack=-0.5)
    try:
        sorter.sort(k, torch.zeros(n, dtype=torch.int32, device=dev))
    except OverflowError:
        Path(f"{out_dir}/overflow{rank}").touch()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_the_single_process_stable_sort(tmp_path):
    import oracle
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    chk = oracle.port()
    for case in ("wide", "narrow", "heavy"):
        in_k = np.concatenate([np.load(tmp_path / f"{case}_in_k{r}.npy") for r in range(world)])
        in_v = np.concatenate([np.load(tmp_path / f"{case}_in_v{r}.npy") for r in range(world)])
        want_k, want_v = chk.sort_by_key(in_k, in_v)
        for exchange in ("nccl", "push"):
            out_k = np.concatenate([np.load(tmp_path / f"{case}_{exchange}_k{r}.npy") for r in range(world)])
            out_v = np.concatenate([np.load(tmp_path / f"{case}_{exchange}_v{r}.npy") for r in range(world)])
            assert out_k.tobytes() == want_k.tobytes(), (case, exchange)
            assert out_v.tobytes() == want_v.tobytes(), (case, exchange)  # stable across ranks
    assert all((tmp_path / f"overflow{r}").exists() for r in range(world))
