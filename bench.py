#!/usr/bin/env python
"""Benchmark of the thrust_b200 hot path.

Headline (one JSON line, rank 0): the sharded stable sort_by_key of (uint64 key,
uint32 value = global index) pairs, 2^30 pairs per GPU, seed 2024 — a plain local
onesweep sort at --gpus 1, the sample sort over NCCL at --gpus 2/4/8 (weak scaling).
`value` is G keys/s of the whole job with inputs resident in HBM; `e2e` is the same
sort through the host-buffer entry point with the H2D / D2H copies inside the timed
region. At --gpus 1 the line also carries `others`: the remaining single-GPU
configurations (int32 sort, float32 / int64 scan, reduce_by_key, (u64,u32) and
(f32,i32) sort_by_key, sort-based histogram), each with its roofline fraction.

`--impl reference` times the reference's own CPU implementation (Thrust 2.2.0 built
with its OMP device system, oracle/_ref) on a bounded sample of the same workload.

`--case NAME [--log2-n N]` runs one small single-GPU case a few times and exits: the
command the profiler captures under profiles/ were taken with (nothing is timed or printed).

Timing: CUDA events on the launching stream, >= 3 warm-up steps, inputs (12 GiB per
GPU) far larger than L2, input restored by a device copy outside the timed events,
max over ranks.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PER_GPU_LOG2 = 30
SEED = 2024
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.file is None:
            return out
        try:
            self.file.flush()
            rows = [r.split(",") for r in Path(self.file.name).read_text().strip().splitlines() if r.count(",") >= 6]
            os.unlink(self.file.name)
        except Exception:
            return out
        sm, reasons = [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                out["sm_max_mhz"] = float(r[1])
            except ValueError:
                continue
            for name, cell in zip(names, r[3:7]):
                if cell.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            busy = [x for x in sm if x >= 0.5 * max(sm)] or sm
            out["sm_mhz"] = statistics.median(busy)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def traffic_per_pair():
    """DRAM bytes per pair and per pass of the onesweep kernel from the committed ncu summary."""
    p = ROOT / "profiles" / "onesweep_traffic.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["dram_bytes_per_pair_per_pass"])
        except Exception:
            return None
    return None


# ------------------------------------------------------------------------------------------
# reference arm: the reference's OMP device system on the host cores
# ------------------------------------------------------------------------------------------
def cpu_sort_sample(log2_n: int, reps: int, warmup: int):
    import numpy as np
    import oracle
    from thrust_b200 import datagen as g
    if oracle.have_ref("omp"):
        chk, kind = oracle.ref("omp"), "reference"
        # all host cores this process may use, whatever OMP_NUM_THREADS the launcher exported
        chk.set_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    else:
        chk, kind = oracle.port(), "port"
        log2_n = min(log2_n, 22)
    n = 1 << log2_n
    keys0 = g.host(g.BITS_U64, n, SEED)
    vals0 = g.host(g.INDEX_U32, n, SEED)
    times = []
    for i in range(warmup + reps):
        k, v = keys0.copy(), vals0.copy()
        t = time.perf_counter()
        chk.sort_by_key_inplace(k, v)
        dt = time.perf_counter() - t
        if i >= warmup:
            times.append(dt)
    assert bool(np.all(k[1:] >= k[:-1]))
    sec = sum(times) / len(times)
    return {
        "value": n / sec / 1e9, "unit": "Gkeys/s", "cores": chk.threads, "kind": kind,
        "sample": f"stable sort_by_key of 2^{log2_n} (uint64 key, uint32 index) pairs, seed {SEED}, "
                  f"Thrust 2.2.0 {'OMP device system' if kind == 'reference' else 'algorithm restated in C'}, "
                  f"mean of {len(times)} runs",
    }, sec


def run_reference(args, rank: int):
    if rank != 0:
        return
    base, sec = cpu_sort_sample(25, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "sort_by_key_throughput", "value": base["value"], "unit": "Gkeys/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "Gkeys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    return {
        "workload": f"sharded stable sort_by_key, 2^{PER_GPU_LOG2} (uint64 key, uint32 value=global index) pairs per GPU, "
                    f"seed {SEED}, {'local onesweep radix sort' if n_gpus == 1 else 'sample sort: regular-sample splitters, stable partition, partition pass storing straight into the receive buffers of the destination GPUs over NVLink (or peer-load gather / NCCL all-to-all), one local onesweep sort'}",
        "pairs_per_gpu": 1 << PER_GPU_LOG2, "total_pairs": n_gpus << PER_GPU_LOG2,
        "l2_policy": "inputs (12 GiB per GPU) larger than L2; input restored by a device copy between steps",
    }


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def time_calls(fn, restore, steps: int, warmup: int, stream):
    """Per-step CUDA-event times (ms) of fn() with restore() run outside the events."""
    import torch
    out = []
    for i in range(warmup + steps):
        restore()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        b.synchronize()
        if i >= warmup:
            out.append(a.elapsed_time(b))
    return out


def _sorted_pairs_ok(k0, v0, k, v, kview=None):
    """Device-side check of a stable sort_by_key whose values were the original indices 0..n-1:
    keys ascending (in `kview` order: an order-preserving integer view of the keys), every output key
    is the input key at its value's index (so the output is a permutation of the input), and equal
    neighbouring keys keep increasing indices (stability)."""
    import torch
    n = k.numel()
    ok = True
    chunk = 1 << 26
    for s in range(0, n, chunk):
        e = min(n, s + chunk + 1)
        kk = k[s:e] if kview is None else kview(k[s:e])
        idx = v[s:e].to(torch.int64) & 0xFFFFFFFF
        ok = ok and bool((kk[1:] >= kk[:-1]).all())
        ok = ok and bool(((kk[1:] != kk[:-1]) | (idx[1:] > idx[:-1])).all())
        ok = ok and bool((k0[idx] == k[s:e]).all())
    return ok


def _u64_order(t):
    """int64 storage of uint64 keys -> int64 values in the same order (flip the sign bit)."""
    return t ^ (-0x8000000000000000)


def _f32_order(t):
    """float32 keys -> int32 values in the bitwise total order the sort uses."""
    import torch
    i = t.view(torch.int32)
    return torch.where(i < 0, i ^ 0x7FFFFFFF, i)


def bench_others(dev, peak):
    """The remaining single-GPU configurations; each entry carries its own roofline fraction and the
    outcome of a device-side check of the last timed result (`verified`)."""
    import torch
    import thrust_b200 as tb
    from thrust_b200 import _capi as capi, datagen as g
    res = {}
    stream = torch.cuda.current_stream(dev)

    def entry(name, fn, restore, units, unit_name, bytes_model, note, verify=None, moved_bytes=None, moved_note=None,
              steps=10):
        try:
            ms = time_calls(fn, restore, steps, 3, stream)
            best, med = min(ms), statistics.median(ms)
            res[name] = {
                "value": units / (med * 1e-3) / 1e9, "unit": unit_name, "ms_median": med, "ms_min": best,
                "algorithmic_GBps": bytes_model / (med * 1e-3) / 1e9,
                "frac_of_hbm_peak": bytes_model / (med * 1e-3) / 1e9 / peak, "bytes_model": note,
            }
            if moved_bytes is not None:  # what the kernels really move, beside the model's figure
                res[name]["moved_GBps"] = moved_bytes / (med * 1e-3) / 1e9
                res[name]["moved_frac_of_hbm_peak"] = moved_bytes / (med * 1e-3) / 1e9 / peak
                res[name]["moved_bytes_model"] = moved_note
            if verify is not None:
                torch.cuda.synchronize(dev)
                res[name]["verified"] = bool(verify())
        except Exception as e:  # keep the headline even if a side configuration fails
            res[name] = {"error": repr(e)}
        torch.cuda.empty_cache()

    # C1: sort of 2^25 int32 keys (working set 128 MiB, partly L2 resident)
    n = 1 << 25
    k0 = g.sort_i32(n, dev)
    k = k0.clone()
    temp = torch.empty(n * 4 + (64 << 20), dtype=torch.uint8, device=dev)

    def c1_ok():
        return bool((k[1:] >= k[:-1]).all()) and int(k.sum()) == int(k0.sum()) and \
            bool((torch.bincount((k & 0xFFFF).to(torch.int64), minlength=1 << 16) ==
                  torch.bincount((k0 & 0xFFFF).to(torch.int64), minlength=1 << 16)).all())
    entry("sort_i32_2^25", lambda: tb.sort(k, sync=False, temp=temp), lambda: k.copy_(k0), n, "Gkeys/s", 48.0 * n,
          "4 passes x (2 reads + 1 write) x 4 B = 48 B/key", verify=c1_ok, moved_bytes=36.0 * n,
          moved_note="one histogram read + 4 passes x (1 read + 1 write) x 4 B = 36 B/key")
    del k, k0, temp

    # C2: scans over 2^30 elements
    n = 1 << 30
    x = g.scan_f32(n, dev)
    y = torch.empty_like(x)
    temp = torch.empty(64 << 20, dtype=torch.uint8, device=dev)

    def scan_ok(exact):
        # prefix sums at a few positions against float64 / int64 sums of the input
        ok = True
        for pos in (0, 1, 10239, 10240, 123456789, n // 2 + 7, n - 1):
            want = x[:pos + 1].sum(dtype=torch.int64 if exact else torch.float64)
            got = y[pos]
            if exact:
                ok = ok and int(got) == int(want)
            else:
                tol = 1e-5 * float(x[:pos + 1].abs().sum(dtype=torch.float64)) + 1e-6
                ok = ok and abs(float(got) - float(want)) <= tol
        return ok
    entry("inclusive_scan_f32_2^30", lambda: tb.inclusive_scan(x, out=y, sync=False, temp=temp), lambda: None,
          n, "Gelem/s", 8.0 * n, "1 read + 1 write x 4 B = 8 B/element", verify=lambda: scan_ok(False))
    # next row of the path: thrust::reduce over the same 2^30 floats (one read)
    red_out = torch.empty(16, dtype=torch.uint8, device=dev)
    red_have = C.c_size_t(temp.numel())
    red_stream = C.c_void_p(stream.cuda_stream)

    def red():
        capi.check(capi.lib.tb200_reduce(C.c_void_p(temp.data_ptr()), C.byref(red_have), C.c_void_p(x.data_ptr()), n,
                                         capi.F32, None, C.c_void_p(red_out.data_ptr()), red_stream), "tb200_reduce")

    def red_ok():
        want = float(x.sum(dtype=torch.float64))
        got = float(red_out[:4].view(torch.float32)[0])
        return abs(got - want) <= 1e-5 * float(x.abs().sum(dtype=torch.float64))
    entry("reduce_f32_2^30", red, lambda: None, n, "Gelem/s", 4.0 * n, "1 read x 4 B = 4 B/element", verify=red_ok)
    del x, y
    x = g.scan_i64(n, dev)
    y = torch.empty_like(x)
    entry("inclusive_scan_i64_2^30", lambda: tb.inclusive_scan(x, out=y, sync=False, temp=temp), lambda: None,
          n, "Gelem/s", 16.0 * n, "1 read + 1 write x 8 B = 16 B/element", verify=lambda: scan_ok(True))
    del x, y

    # C2: reduce_by_key over 2^28 grouped keys, mean run 16
    n = 1 << 28
    keys, vals = g.rbk_inputs(n, dev)
    ko, vo = torch.empty_like(keys), torch.empty_like(vals)
    runs = torch.zeros(1, dtype=torch.int64, device=dev)
    st = C.c_void_p(stream.cuda_stream)
    have = C.c_size_t(temp.numel())

    def rbk():
        capi.check(capi.lib.tb200_reduce_by_key(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()),
            C.c_void_p(ko.data_ptr()), C.c_void_p(vo.data_ptr()), C.c_void_p(runs.data_ptr()), n, capi.I32, capi.F32,
            st), "tb200_reduce_by_key")
    rbk()
    nruns = int(runs.item())
    # keys are run ids 0..runs-1 (already grouped): per-run sums in float64 are one index_add away
    run_of = keys.to(torch.int64)

    def seg_sums(v):
        out = torch.zeros(int(run_of[-1]) + 1, dtype=torch.float64, device=dev)
        for s in range(0, n, 1 << 26):
            out.index_add_(0, run_of[s:s + (1 << 26)], v[s:s + (1 << 26)].to(torch.float64))
        return out

    def rbk_ok():
        want, wabs = seg_sums(vals), seg_sums(vals.abs())
        r = int(runs.item())
        return r == want.numel() and bool((ko[:r] == torch.arange(r, dtype=torch.int32, device=dev)).all()) and \
            bool(((vo[:r].to(torch.float64) - want).abs() <= 1e-5 * wabs + 1e-30).all())
    entry("reduce_by_key_i32_f32_2^28", rbk, lambda: None, n, "Gelem/s", 8.0 * (n + nruns),
          f"(n + runs) x (4 B key + 4 B value), runs = {nruns}", verify=rbk_ok)
    # next row of the path: inclusive_scan_by_key over the same keys and values
    so = torch.empty_like(vals)

    def sbk():
        capi.check(capi.lib.tb200_scan_by_key(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()),
            C.c_void_p(so.data_ptr()), n, capi.I32, capi.F32, 0, None, st), "tb200_scan_by_key")

    def sbk_ok():
        # the last element of every run holds the run's sum; the first holds its own value
        want, wabs = seg_sums(vals), seg_sums(vals.abs())
        last = torch.ones(n, dtype=torch.bool, device=dev)
        last[:-1] = keys[1:] != keys[:-1]
        first = torch.ones(n, dtype=torch.bool, device=dev)
        first[1:] = last[:-1]
        return bool(((so[last].to(torch.float64) - want).abs() <= 1e-5 * wabs + 1e-30).all()) and \
            bool((so[first] == vals[first]).all())
    entry("inclusive_scan_by_key_i32_f32_2^28", sbk, lambda: None, n, "Gelem/s", 12.0 * n,
          "4 B key + 4 B value read, 4 B value written = 12 B/element", verify=sbk_ok)
    # next row of the path: unique_by_key_copy over the same keys and values
    kept = torch.zeros(1, dtype=torch.int64, device=dev)

    def ubk():
        capi.check(capi.lib.tb200_unique_by_key(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()),
            C.c_void_p(ko.data_ptr()), C.c_void_p(vo.data_ptr()), C.c_void_p(kept.data_ptr()), n, capi.I32, 4, st),
            "tb200_unique_by_key")

    def ubk_ok():
        first = torch.ones(n, dtype=torch.bool, device=dev)
        first[1:] = keys[1:] != keys[:-1]
        r = int(kept.item())
        return r == int(first.sum()) and bool((ko[:r] == keys[first]).all()) and bool((vo[:r] == vals[first]).all())
    entry("unique_by_key_i32_f32_2^28", ubk, lambda: None, n, "Gelem/s", 8.0 * (n + nruns),
          f"(n + kept) x (4 B key + 4 B value), kept = {nruns}", verify=ubk_ok)
    # next row of the path: copy_if with a stencil (half of the 4-byte elements selected)
    flags = (keys & 1).to(torch.uint8)  # the low bit of the run id: whole runs in or out, about half of the elements
    nsel = int(flags.sum())

    def cpf():
        capi.check(capi.lib.tb200_copy_flagged(
            C.c_void_p(temp.data_ptr()), C.byref(have), C.c_void_p(vals.data_ptr()), C.c_void_p(flags.data_ptr()),
            C.c_void_p(vo.data_ptr()), C.c_void_p(kept.data_ptr()), n, 4, capi.U8, st), "tb200_copy_flagged")

    def cpf_ok():
        r = int(kept.item())
        return r == nsel and bool((vo[:r] == vals[flags.bool()]).all())
    entry("copy_if_stencil_f32_u8_2^28", cpf, lambda: None, n, "Gelem/s", 5.0 * n + 4.0 * nsel,
          f"4 B element + 1 B flag read, 4 B written per selected element, selected = {nsel}", verify=cpf_ok)
    del keys, vals, ko, vo, so, run_of, flags

    # C3: stable sort_by_key of 2^28 (uint64, uint32) pairs
    k0, v0 = g.pairs_u64_u32(n, g.SEED_PAIRS_U64, 0, dev)
    k, v = k0.clone(), v0.clone()
    temp = torch.empty(n * 12 + (128 << 20), dtype=torch.uint8, device=dev)
    entry("sort_by_key_u64_u32_2^28", lambda: tb.sort_by_key(k, v, key_dtype=capi.U64, sync=False, temp=temp),
          lambda: (k.copy_(k0), v.copy_(v0)), n, "Gkeys/s", 256.0 * n,
          "8 passes x (3 x 8 B key + 2 x 4 B value) = 256 B/pair",
          verify=lambda: _sorted_pairs_ok(k0, v0, k, v, _u64_order), moved_bytes=200.0 * n,
          moved_note="one histogram read (8 B) + 8 passes x (1 read + 1 write) x 12 B = 200 B/pair")
    del k, v, k0, v0

    # C4: (float32, int32) pairs, low entropy
    k0, v0 = g.and3_pairs(n, dev)
    k, v = k0.clone(), v0.clone()
    entry("sort_by_key_f32_i32_and3_2^28", lambda: tb.sort_by_key(k, v, sync=False, temp=temp),
          lambda: (k.copy_(k0), v.copy_(v0)), n, "Gkeys/s", 80.0 * n,
          "4 passes x (3 x 4 B key + 2 x 4 B value) = 80 B/pair",
          verify=lambda: _sorted_pairs_ok(k0.view(torch.int32), v0, k.view(torch.int32), v, _f32_order_i32),
          moved_bytes=68.0 * n, moved_note="one histogram read (4 B) + 4 passes x (1 read + 1 write) x 8 B = 68 B/pair")
    del k0, v0
    k0, v0, table = g.zipf_pairs(n, dev)
    entry("sort_by_key_f32_i32_zipf_2^28", lambda: tb.sort_by_key(k, v, sync=False, temp=temp),
          lambda: (k.copy_(k0), v.copy_(v0)), n, "Gkeys/s", 80.0 * n,
          "4 passes x (3 x 4 B key + 2 x 4 B value) = 80 B/pair",
          verify=lambda: _sorted_pairs_ok(k0.view(torch.int32), v0, k.view(torch.int32), v, _f32_order_i32),
          moved_bytes=68.0 * n, moved_note="one histogram read (4 B) + up to 4 passes x (1 read + 1 write) x 8 B = 68 B/pair")
    counts_box = [None]

    def hist():
        tb.sort(k, sync=False, temp=temp)
        counts_box[0] = tb.histogram_sorted(k, table, sync=False)

    def hist_ok():
        # the keys are table[rank]: recover every key's rank by search and count the ranks
        want = torch.zeros(table.numel(), dtype=torch.int64, device=dev)
        for s in range(0, n, 1 << 26):
            want += torch.bincount(torch.searchsorted(table, k0[s:s + (1 << 26)]), minlength=table.numel())
        got = counts_box[0].to(torch.int64) & 0xFFFFFFFF
        return bool((got == want).all()) and int(got.sum()) == n
    entry("dense_histogram_zipf_f32_65536_bins_2^28", hist, lambda: k.copy_(k0), n, "Gkeys/s", 48.0 * n,
          "keys-only sort: 4 passes x 12 B = 48 B/key (search + difference touch < 1 MB)", verify=hist_ok,
          moved_bytes=36.0 * n, moved_note="one histogram read + up to 4 passes x (1 read + 1 write) x 4 B = 36 B/key")
    return res


def _f32_order_i32(i):
    """int32 view of float32 keys -> int32 values in the bitwise total order the sort uses."""
    import torch
    return torch.where(i < 0, i ^ 0x7FFFFFFF, i)


CASES = ("sort_u64_u32", "sort_i32", "sort_f32_i32", "scan_f32", "scan_i64", "reduce_by_key", "scan_by_key",
         "unique_by_key", "copy_flagged", "reduce_f32", "histogram_f32", "partition_u64_u32")


def run_case(case: str, log2_n: int, reps: int = 3) -> None:
    """One small single-GPU case for a profiler capture: seeded input generated on the device
    (larger than L2 from log2_n = 26, well under a few GB), the algorithm run `reps` times through
    the C ABI."""
    import torch
    import thrust_b200 as tb
    from thrust_b200 import _capi as capi, datagen as g
    n = 1 << log2_n
    dev = torch.device("cuda:0")
    if case == "sort_u64_u32":
        k0, v0 = g.pairs_u64_u32(n, SEED, 0, dev)
        for _ in range(reps):
            k, v = k0.clone(), v0.clone()
            tb.sort_by_key(k, v, key_dtype=capi.U64)
    elif case == "sort_i32":
        k0 = g.sort_i32(n, dev)
        for _ in range(reps):
            k = k0.clone()
            tb.sort(k)
    elif case == "sort_f32_i32":
        k0, v0 = g.and3_pairs(n, dev)
        for _ in range(reps):
            k, v = k0.clone(), v0.clone()
            tb.sort_by_key(k, v)
    elif case in ("scan_f32", "scan_i64"):
        x = g.scan_f32(n, dev) if case == "scan_f32" else g.scan_i64(n, dev)
        y = torch.empty_like(x)
        for _ in range(reps):
            tb.inclusive_scan(x, out=y)
    elif case in ("reduce_by_key", "scan_by_key", "unique_by_key", "copy_flagged"):
        k, v = g.rbk_inputs(n, dev)
        out = torch.empty_like(v)
        flags = (k & 1).to(torch.uint8)
        for _ in range(reps):
            if case == "reduce_by_key":
                tb.reduce_by_key(k, v)
            elif case == "scan_by_key":
                tb.inclusive_scan_by_key(k, v, out=out)
            elif case == "unique_by_key":
                tb.unique_by_key(k, v)
            else:
                tb.copy_flagged(v, flags, out=out)
    elif case == "reduce_f32":
        x = g.scan_f32(n, dev)
        for _ in range(reps):
            tb.reduce(x)
    elif case == "histogram_f32":
        k0, _, table = g.zipf_pairs(n, dev)
        for _ in range(reps):
            tb.dense_histogram(k0, table)
    elif case == "partition_u64_u32":
        from thrust_b200 import sample_sort as ss
        k0, v0 = g.pairs_u64_u32(n, SEED, 0, dev)
        ops = ss.DeviceOps(dev, n)
        splitters = (torch.arange(1, 8, dtype=torch.int64, device=dev) << 61)
        ok, ov = torch.empty_like(k0), torch.empty_like(v0)
        for _ in range(reps):
            ops.partition(k0, v0, n, splitters, ok, ov)
    else:
        raise SystemExit(f"unknown case {case!r}; one of {', '.join(CASES)}")
    torch.cuda.synchronize()
    print("done", case, n)


def cpp_policy_timing():
    """Times thrust::sort(thrust_b200::par, ...) on 2^25 int32 keys from the C++ side (pool lease,
    launches, status read-back included): tests/cpp/bin/bench_system prints one JSON object."""
    exe = ROOT / "tests" / "cpp" / "bin" / "bench_system"
    if not exe.exists():
        return None
    try:
        r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
        return json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 else {"error": r.stderr[-300:]}
    except Exception as e:
        return {"error": repr(e)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2-per-gpu", type=int, default=PER_GPU_LOG2, help="for quick checks only")
    ap.add_argument("--no-others", action="store_true", help="skip the side configurations at --gpus 1")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--engine", default="python", choices=["python", "c"],
                    help="who runs the steps of the sharded sort at --gpus > 1: the Python class over torch.distributed, "
                         "or one call of the C entry point tb200_sample_sort on its own NCCL communicator")
    ap.add_argument("--exchange", default="auto", choices=["auto", "push", "peer", "nccl"],
                    help="exchange step of the sharded sort at --gpus > 1 (default: push over NVLink)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--case", default=None, help=f"run one small case for a profiler and exit: {', '.join(CASES)}")
    ap.add_argument("--log2-n", type=int, default=26, help="size of --case (default 2^26 elements)")
    args = ap.parse_args()
    if args.case is not None:
        run_case(args.case, args.log2_n)
        return
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import thrust_b200 as tb
    from thrust_b200 import _capi as capi, datagen as g, sample_sort as ss

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: thrust_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peak, peak_kind = measured_peak()
    n = 1 << args.log2_per_gpu
    stream = torch.cuda.current_stream(dev)

    sorter = ss.ShardedSorter(n, dev, world_size=world, rank=rank, seed=SEED, exchange=args.exchange,
                              engine=args.engine)
    k0, v0 = g.pairs_u64_u32(n, SEED, rank * n, dev)
    k, v = torch.empty_like(k0), torch.empty_like(v0)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    step_ms, trace_ms = [], []
    ms_buf = (C.c_float * 64)()
    kind_buf = (C.c_int * 64)()
    for i in range(args.warmup):
        k.copy_(k0); v.copy_(v0)
        sorter.sort(k, v)
    barrier()
    with ClockSampler(local_rank) as clocks:
        for i in range(args.steps):
            k.copy_(k0); v.copy_(v0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world > 1:
                dist.barrier()
            capi.lib.tb200_trace_begin(C.c_void_p(stream.cuda_stream))
            a.record(stream)
            out_k, out_v, out_n = sorter.sort(k, v)
            b.record(stream)
            b.synchronize()
            cnt = capi.lib.tb200_trace_end(ms_buf, kind_buf, 64)
            step_ms.append(a.elapsed_time(b))
            trace_ms.append([(kind_buf[j], ms_buf[j]) for j in range(max(min(cnt, 64), 0))])
        barrier()
    sorter.check_status()
    phases = sorter.phase_times()
    sorter_exchange = sorter.exchange
    ok = sorter.verify(out_k, out_v, out_n)

    t = torch.tensor(step_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms = t.tolist()
    ms_per_step = sum(step_ms) / len(step_ms)
    total_pairs = n * world
    value = total_pairs / (ms_per_step * 1e-3) / 1e9

    # dominant kernel: one onesweep radix pass (trace kind 2) over this rank's pairs. At N > 1 the
    # passes run over the received pairs (about n of them), so n is used for every launch.
    # (the last 8 radix passes of a step: at N > 1 the splitter sample is sorted first, with tiny passes)
    pass_ms = [ms for tr in trace_ms for ms in [m for kind, m in tr if kind == 2][-8:]]
    avg_pass = sum(pass_ms) / max(len(pass_ms), 1)
    pass_bytes = n * 2.0 * (8 + 4)
    achieved = pass_bytes / (avg_pass * 1e-3) / 1e9 if avg_pass > 0 else 0.0
    tpp = traffic_per_pair()
    def last_sort(tr):  # launches of the last local sort of a step: histogram, passes, copy-back
        idx = [i for i, (kind, _) in enumerate(tr) if kind == 1]
        return tr[idx[-1]:] if idx else []
    sort_ms = [sum(ms for kind, ms in last_sort(tr) if kind in (1, 2, 3)) for tr in trace_ms]
    whole = (256.0 * n) / (sum(sort_ms) / max(len(sort_ms), 1) * 1e-3) / 1e9 if sort_ms and sort_ms[0] > 0 else None
    roofline = {
        "bound": "hbm", "kernel": "onesweep_kernel<u64 key, 4-byte value>", "achieved": achieved, "peak": peak,
        "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
        "traffic": None if tpp is None else tpp * n, "algorithmic_bytes_per_launch": pass_bytes,
        "avg_launch_ms": avg_pass, "launches_timed": len(pass_ms),
        "whole_sort_3touch": {
            "bytes_per_pair": 256, "model": "8 passes x (2 reads + 1 write of an 8 B key, 1 read + 1 write of a 4 B value)",
            "achieved": whole, "frac": None if whole is None else whole / peak,
            "note": "local sort only (histogram + 8 passes + copy-back launches)",
        },
    }
    launches = sum(len(tr) for tr in trace_ms)

    del k0, v0, k, v, out_k, out_v
    sorter.release()
    torch.cuda.empty_cache()

    e2e = None
    if not args.no_e2e:
        e2e = ss.bench_host_path(n, dev, world, rank, SEED, steps=min(args.steps, 3), warmup=1)

    line = {
        "metric": "sort_by_key_throughput", "value": value, "unit": "Gkeys/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u64", "data": "synthetic", "config": workload_config(world),
        "verified": bool(ok), "clocks": clocks.summary(), "roofline": roofline, "gpu_launches": launches,
        "e2e": e2e,
    }
    if world > 1:
        line["phases_ms_rank0_last_step"] = phases
        line["config"]["exchange"] = sorter_exchange
        line["config"]["engine"] = args.engine
    if rank == 0 and world == 1:
        if not args.no_cpu:
            line["cpu_baseline"], _ = cpu_sort_sample(25, 3, 1)
        if not args.no_others:
            line["others"] = bench_others(dev, peak)
            cpp = cpp_policy_timing()
            if cpp is not None:
                line["others"]["thrust_sort_through_policy_i32_2^25"] = cpp
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
