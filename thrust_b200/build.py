"""Build the CUDA library of this package for sm_100a, in-tree.

`python -m thrust_b200.build` compiles every `csrc/*.cu` with nvcc
(`-gencode arch=compute_100a,code=sm_100a`) and links `libthrust_b200.so` next
to this file. Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libthrust_b200.so"
# test / benchmark support (seeded inputs, reference-free checker): its own library
DATAGEN_SRC = PKG / "datagen" / "datagen.cu"
DATAGEN_LIB = PKG / "datagen" / "libtb200_datagen.so"
# the sharded sort behind one C entry point: links NCCL, so it is a library of its own
NCCL_SRC = PKG / "csrc_nccl" / "sample_sort.cu"
NCCL_LIB = PKG / "libthrust_b200_nccl.so"
ROOT = PKG.parent

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-ccbin", "/usr/bin/g++",
    "-Xcompiler", "-fPIC,-O3,-fopenmp", "-I", str(ROOT / "include"),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library of thrust_b200 cannot be built")
    return exe


def _newest_header() -> float:
    hs = (list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").rglob("*.h")) +
          list(DATAGEN_SRC.parent.glob("*.h")))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, verbose: bool, obj_dir: Path = OBJ, extra=()) -> Path:
    obj = obj_dir / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose and r.stderr:
        (obj_dir / (src.stem + ".ptxas.txt")).write_text(r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link; returns the path of the shared library."""
    OBJ.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    hdr_time = _newest_header()
    todo = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_time):
            todo.append(s)
    dg_obj = OBJ / (DATAGEN_SRC.stem + ".o")
    dg_stale = force or not dg_obj.exists() or dg_obj.stat().st_mtime < max(DATAGEN_SRC.stat().st_mtime, hdr_time)
    work = todo + ([DATAGEN_SRC] if dg_stale else [])
    if work:
        with cf.ThreadPoolExecutor(max_workers=min(len(work), os.cpu_count() or 4)) as ex:
            list(ex.map(lambda s: _compile(s, verbose), work))
    if dg_stale or not DATAGEN_LIB.exists():
        cmd = [_nvcc(), "-shared", "-o", str(DATAGEN_LIB), str(dg_obj), "-ccbin", "/usr/bin/g++", "-lcudart", "-lgomp"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if todo or not LIB.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-ccbin", "/usr/bin/g++", "-lcudart", "-lgomp"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    nccl_obj = OBJ / "nccl_sample_sort.o"
    if force or not NCCL_LIB.exists() or NCCL_LIB.stat().st_mtime < max(NCCL_SRC.stat().st_mtime, hdr_time, LIB.stat().st_mtime):
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(NCCL_SRC), "-o", str(nccl_obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {NCCL_SRC.name} (needs nccl.h):\n{r.stdout}\n{r.stderr}")
        cmd = [_nvcc(), "-shared", "-o", str(NCCL_LIB), str(nccl_obj), "-ccbin", "/usr/bin/g++", "-L", str(PKG),
               "-lthrust_b200", "-lnccl", "-lcudart", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
