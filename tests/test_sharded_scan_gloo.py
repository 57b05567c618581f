"""Host-side logic of the sharded scan and the sharded reduce_by_key over gloo, world size 2
and 3, on CPU.

The per-shard compute is injected (a numpy `ops` object backed by the CPU oracle), so these
tests exercise exactly the orchestration the GPU path runs: the exchange of the shard totals and
the seeds, and the hand-over of runs that cross shard boundaries (empty shards, shards that lie
inside one run, runs over three ranks) — and compare the concatenated result with the oracle on
the concatenated input.
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
    """CPU stand-in for ScanOps: same methods, the oracle's sequential algorithms."""

    def __init__(self):
        import oracle
        self.chk = oracle.port()

    def reduce(self, x):
        a = x.numpy()
        return self.chk.scan(a)[-1].item() if a.size else 0

    def scan(self, x, out, exclusive, seed):
        a = x.numpy()
        if exclusive:
            res = self.chk.scan(a, True, seed)
        else:  # seeded inclusive scan: the exclusive one shifted by the element itself
            with np.errstate(over="ignore"):
                res = (self.chk.scan(a, True, seed) + a).astype(a.dtype)
        out.copy_(torch.from_numpy(res))

    def reduce_by_key(self, keys, vals):
        ko, vo = self.chk.reduce_by_key(keys.numpy(), vals.numpy())
        return torch.from_numpy(ko.copy()), torch.from_numpy(vo.copy()), int(ko.size)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _shard_sizes(world, case):
    return {"even": [3000] * world, "ragged": [2500, 0, 3100][:world] if world == 3 else [0, 4000],
            "tiny": [1, 2, 1][:world]}[case]


def _worker(rank, world, port, case, vdtype, p_new, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from thrust_b200.sharded_scan import ShardedScan
    sizes = _shard_sizes(world, case)
    rng = np.random.default_rng(77)  # every rank draws the whole input and keeps its shard
    n = sum(sizes)
    heads = rng.random(n) < p_new
    keys = (np.cumsum(heads) % 5).astype(np.int32)  # equal keys come back: runs, not groups
    if np.issubdtype(vdtype, np.integer):
        ii = np.iinfo(vdtype)
        vals = rng.integers(ii.min, ii.max, size=n, dtype=vdtype, endpoint=True)  # sums wrap
    else:
        vals = rng.uniform(-50, 50, size=n).astype(vdtype)
    lo = sum(sizes[:rank])
    k, v = keys[lo:lo + sizes[rank]].copy(), vals[lo:lo + sizes[rank]].copy()
    if rank == 0:
        np.save(f"{out_dir}/keys.npy", keys)
        np.save(f"{out_dir}/vals.npy", vals)
    sh = ShardedScan(world, rank, ops=OracleOps())
    tv = torch.from_numpy(v)
    np.save(f"{out_dir}/inc{rank}.npy", sh.inclusive_scan(tv).numpy())
    np.save(f"{out_dir}/exc{rank}.npy", sh.exclusive_scan(tv, init=7).numpy())
    ko, vo, m = sh.reduce_by_key(torch.from_numpy(k), tv)
    np.save(f"{out_dir}/rk{rank}.npy", ko[:m].numpy())
    np.save(f"{out_dir}/rv{rank}.npy", vo[:m].numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,case,vdtype,p_new", [
    (2, "even", np.int32, 1 / 16), (3, "even", np.int64, 0.0004), (3, "ragged", np.int32, 0.001),
    (2, "ragged", np.int64, 1 / 3), (3, "tiny", np.int32, 0.0), (3, "even", np.float32, 1 / 16),
    (2, "even", np.float64, 0.0002)])
def test_sharded_scan_and_reduce_by_key_match_the_oracle_on_the_whole_input(tmp_path, world, case, vdtype, p_new):
    import oracle
    oracle.build(ref=False)
    port = _free_port()
    mp.spawn(_worker, args=(world, port, case, vdtype, p_new, str(tmp_path)), nprocs=world, join=True)
    keys, vals = np.load(tmp_path / "keys.npy"), np.load(tmp_path / "vals.npy")
    chk = oracle.port()
    cat = lambda stem: np.concatenate([np.load(tmp_path / f"{stem}{r}.npy") for r in range(world)])
    want_k, want_v = chk.reduce_by_key(keys, vals)
    got_k, got_v = cat("rk"), cat("rv")
    assert got_k.tobytes() == want_k.tobytes()
    if np.issubdtype(vdtype, np.integer):  # bit-exact: wrapping sums are associative
        assert cat("inc").tobytes() == chk.scan(vals).tobytes()
        assert cat("exc").tobytes() == chk.scan(vals, True, 7).tobytes()
        assert got_v.tobytes() == want_v.tobytes()
    else:  # another grouping of the same sum: within 1e-5 of the sum of magnitudes
        tol = 1e-5 * float(np.abs(vals.astype(np.float64)).sum()) + 1e-30
        assert float(np.max(np.abs(cat("inc").astype(np.float64) - chk.scan(vals).astype(np.float64)))) <= tol
        assert float(np.max(np.abs(cat("exc").astype(np.float64) - chk.scan(vals, True, 7).astype(np.float64)))) <= tol
        assert float(np.max(np.abs(got_v.astype(np.float64) - want_v.astype(np.float64)))) <= tol
