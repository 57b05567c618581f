"""Build the C++ boundary test (Thrust custom system over the C ABI) and the small C++ timing
program of the policy path for sm_100a.

Output: tests/cpp/bin/test_system, bench_system and test_sample_sort (the C entry point of the
sharded sort called from C++), linked against thrust_b200/libthrust_b200.so by relative rpath. Uses the CUDA toolkit's Thrust headers.
"""
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
LIBDIR = ROOT / "thrust_b200"
PROGRAMS = ("test_system", "bench_system", "test_sample_sort")


def _build_one(name: str, force: bool) -> Path:
    src, out = HERE / f"{name}.cu", HERE / "bin" / name
    deps = [src, ROOT / "include" / "thrust_b200" / "system.h", ROOT / "include" / "thrust_b200.h"]
    if not force and out.exists() and out.stat().st_mtime >= max(d.stat().st_mtime for d in deps):
        return out
    out.parent.mkdir(exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
           "--extended-lambda", "-ccbin", "/usr/bin/g++", "-I", str(ROOT / "include"), str(src), "-o", str(out),
           "-L", str(LIBDIR), "-lthrust_b200", "-Xlinker", "-rpath=$ORIGIN/../../../thrust_b200"]
    if name == "test_sample_sort":  # the sharded sort's C entry point lives in the NCCL library
        cmd += ["-lthrust_b200_nccl", "-lnccl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n" + r.stdout + r.stderr)
    return out


def build(force: bool = False) -> Path:
    outs = [_build_one(name, force) for name in PROGRAMS]
    return outs[0]


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
