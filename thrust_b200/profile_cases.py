"""Small single-GPU cases for profiler captures.

    python -m thrust_b200.profile_cases <case> [log2_n]

cases: sort_u64_u32, sort_i32, sort_f32_i32, scan_f32, scan_i64, reduce_by_key, scan_by_key,
reduce_f32.
Each case generates its seeded input on the device (larger than L2 from log2_n = 26),
runs the algorithm a few times through the C ABI and exits; it holds well under a few GB,
which is what a multi-pass profiler capture needs.
"""
from __future__ import annotations

import sys

import torch

from . import _capi as capi
from . import algorithms as alg
from . import datagen as g


def run(case: str, log2_n: int = 26, reps: int = 3) -> None:
    n = 1 << log2_n
    dev = torch.device("cuda:0")
    if case == "sort_u64_u32":
        k0, v0 = g.pairs_u64_u32(n, g.SEED_SHARDED, 0, dev)
        for _ in range(reps):
            k, v = k0.clone(), v0.clone()
            alg.sort_by_key(k, v, key_dtype=capi.U64)
    elif case == "sort_i32":
        k0 = g.sort_i32(n, dev)
        for _ in range(reps):
            k = k0.clone()
            alg.sort(k)
    elif case == "sort_f32_i32":
        k0, v0 = g.and3_pairs(n, dev)
        for _ in range(reps):
            k, v = k0.clone(), v0.clone()
            alg.sort_by_key(k, v)
    elif case in ("scan_f32", "scan_i64"):
        x = g.scan_f32(n, dev) if case == "scan_f32" else g.scan_i64(n, dev)
        y = torch.empty_like(x)
        for _ in range(reps):
            alg.inclusive_scan(x, out=y)
    elif case == "reduce_by_key":
        k, v = g.rbk_inputs(n, dev)
        for _ in range(reps):
            alg.reduce_by_key(k, v)
    elif case == "scan_by_key":
        k, v = g.rbk_inputs(n, dev)
        out = torch.empty_like(v)
        for _ in range(reps):
            alg.inclusive_scan_by_key(k, v, out=out)
    elif case == "reduce_f32":
        x = g.scan_f32(n, dev)
        for _ in range(reps):
            alg.reduce(x)
    else:
        raise SystemExit(f"unknown case {case!r}")
    torch.cuda.synchronize()
    print("done", case, n)


if __name__ == "__main__":
    run(sys.argv[1], int(sys.argv[2]) if len(sys.argv) > 2 else 26)
