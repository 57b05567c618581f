"""Sharded scan and reduce_by_key on two GPUs over NCCL (one process per GPU), against the oracle
on the concatenated input. Skipped on boxes with one GPU; the host logic alone is covered on CPU
ranks by test_sharded_scan_gloo.py."""
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
    from thrust_b200.sharded_scan import ShardedScan
    sizes = [1_000_003, 700_001]
    n = sum(sizes)
    rng = np.random.default_rng(2024)  # every rank draws the whole input and keeps its shard
    keys = np.cumsum(rng.random(n) < 0.00002).astype(np.int32)  # long runs: some cross the shard boundary
    vals = rng.integers(-1000, 1000, size=n, dtype=np.int64)
    lo = sum(sizes[:rank])
    k = torch.from_numpy(keys[lo:lo + sizes[rank]].copy()).to(dev)
    v = torch.from_numpy(vals[lo:lo + sizes[rank]].copy()).to(dev)
    if rank == 0:
        np.save(f"{out_dir}/keys.npy", keys)
        np.save(f"{out_dir}/vals.npy", vals)
    sh = ShardedScan(world, rank)
    np.save(f"{out_dir}/inc{rank}.npy", sh.inclusive_scan(v).cpu().numpy())
    np.save(f"{out_dir}/exc{rank}.npy", sh.exclusive_scan(v, init=-5).cpu().numpy())
    ko, vo, m = sh.reduce_by_key(k, v)
    np.save(f"{out_dir}/rk{rank}.npy", ko[:m].cpu().numpy())
    np.save(f"{out_dir}/rv{rank}.npy", vo[:m].cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_the_oracle_on_the_whole_input(tmp_path):
    import oracle
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    keys, vals = np.load(tmp_path / "keys.npy"), np.load(tmp_path / "vals.npy")
    chk = oracle.port()
    cat = lambda stem: np.concatenate([np.load(tmp_path / f"{stem}{r}.npy") for r in range(world)])
    assert cat("inc").tobytes() == chk.scan(vals).tobytes()
    assert cat("exc").tobytes() == chk.scan(vals, True, -5).tobytes()
    wk, wv = chk.reduce_by_key(keys, vals)
    assert cat("rk").tobytes() == wk.tobytes() and cat("rv").tobytes() == wv.tobytes()
