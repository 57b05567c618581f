"""Build the C++ boundary test (Thrust custom system over the C ABI) for sm_100a.

Output: tests/cpp/bin/test_system, linked against thrust_b200/libthrust_b200.so by
relative rpath. Uses the CUDA toolkit's Thrust headers.
"""
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
SRC = HERE / "test_system.cu"
OUT = HERE / "bin" / "test_system"
LIBDIR = ROOT / "thrust_b200"


def build(force: bool = False) -> Path:
    deps = [SRC, ROOT / "include" / "thrust_b200" / "system.h", ROOT / "include" / "thrust_b200.h"]
    if not force and OUT.exists() and OUT.stat().st_mtime >= max(d.stat().st_mtime for d in deps):
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
           "--extended-lambda", "-ccbin", "/usr/bin/g++", "-I", str(ROOT / "include"), str(SRC), "-o", str(OUT),
           "-L", str(LIBDIR), "-lthrust_b200", "-Xlinker", "-rpath=$ORIGIN/../../../thrust_b200"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for test_system.cu:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
