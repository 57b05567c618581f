"""TEST INFRASTRUCTURE — CPU checkers for thrust_b200. Never imported by the product.

Two interchangeable checkers with the same numpy-facing methods:

* ``port()``      — oracle/liboracle.so, the plain-C restatement (oracle.c);
* ``ref("omp")`` / ``ref("cpp")`` — oracle/_ref/libthrust_ref_*.so, the unmodified
  reference headers compiled against the reference's own OMP / CPP device system
  (ref_shim.cpp). Built where the reference tree exists; the built files travel.

Only tests/, ``__graft_entry__.smoke()`` and bench.py's CPU-baseline legs may import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path
from typing import Optional, Tuple

import numpy as np

HERE = Path(__file__).resolve().parent

I8, U8, I16, U16, I32, U32, I64, U64, F32, F64, BOOL = range(11)
_NP_TO_DT = {
    np.dtype(np.int8): I8, np.dtype(np.uint8): U8, np.dtype(np.int16): I16, np.dtype(np.uint16): U16,
    np.dtype(np.int32): I32, np.dtype(np.uint32): U32, np.dtype(np.int64): I64, np.dtype(np.uint64): U64,
    np.dtype(np.float32): F32, np.dtype(np.float64): F64, np.dtype(np.bool_): BOOL,
}


def dt_of(a: np.ndarray) -> int:
    return _NP_TO_DT[a.dtype]


def reference_tree() -> Path:
    """Where the reference project is looked for: $REF, else the Makefile's default."""
    return Path(os.environ.get("REF", "/root/reference"))


def build(ref: bool = True) -> None:
    """Compile liboracle.so and, when the reference tree is present, oracle/_ref."""
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    tree = reference_tree()
    if ref and (tree / "thrust" / "version.h").exists():
        subprocess.run(["make", "-s", "-j2", "-C", str(HERE), "ref", f"REF={tree}"], check=True)


class CpuChecker:
    """numpy front end over one of the CPU libraries (prefix ``oracle_`` or ``ref_``)."""

    def __init__(self, path: Path, prefix: str, kind: str):
        if not path.exists():
            raise FileNotFoundError(f"{path} not built (run `make -C oracle`)")
        self.kind = kind
        self.path = path
        self._lib = C.CDLL(str(path))
        vp, u64, i32, u32 = C.c_void_p, C.c_uint64, C.c_int, C.c_uint32
        self._sort = getattr(self._lib, prefix + "sort")
        self._sort.argtypes, self._sort.restype = [vp, u64, i32, i32], i32
        self._sbk = getattr(self._lib, prefix + "sort_by_key")
        self._sbk.argtypes, self._sbk.restype = [vp, vp, u64, i32, i32, i32], i32
        self._scan = getattr(self._lib, prefix + "scan")
        self._scan.argtypes, self._scan.restype = [vp, vp, u64, i32, i32, vp], i32
        self._rbk = getattr(self._lib, prefix + "reduce_by_key")
        self._rbk.argtypes, self._rbk.restype = [vp, vp, vp, vp, u64, i32, i32], C.c_int64
        self._sbk_scan = getattr(self._lib, prefix + "scan_by_key")
        self._sbk_scan.argtypes, self._sbk_scan.restype = [vp, vp, vp, u64, i32, i32, i32, vp], i32
        self._reduce = getattr(self._lib, prefix + "reduce")
        self._reduce.argtypes, self._reduce.restype = [vp, u64, i32, vp, vp], i32
        self._hist = getattr(self._lib, prefix + "histogram")
        self._hist.argtypes, self._hist.restype = [vp, u64, i32, vp, u32, vp], i32
        self._ubk = getattr(self._lib, prefix + "unique_by_key")
        self._ubk.argtypes, self._ubk.restype = [vp, vp, vp, vp, u64, i32, i32], C.c_int64
        self._cpf = getattr(self._lib, prefix + "copy_flagged")
        self._cpf.argtypes, self._cpf.restype = [vp, vp, vp, u64, i32, i32], C.c_int64
        self.threads = 1
        if prefix == "ref_":
            self._lib.ref_num_threads.restype = i32
            self.threads = int(self._lib.ref_num_threads())
            self._lib.ref_thrust_version.restype = i32
            self.thrust_version = int(self._lib.ref_thrust_version())

    def set_threads(self, n: int) -> int:
        """Asks the OMP reference library for n threads (no-op for the others); returns the count in use."""
        if hasattr(self._lib, "ref_set_num_threads") and self.kind != "port":
            try:
                self._lib.ref_set_num_threads.argtypes = [C.c_int]
                self._lib.ref_set_num_threads(int(n))
                self.threads = int(self._lib.ref_num_threads())
            except AttributeError:
                pass
        return self.threads

    @staticmethod
    def _p(a: Optional[np.ndarray]):
        return None if a is None else C.c_void_p(a.ctypes.data)

    def sort(self, keys: np.ndarray, descending: bool = False) -> np.ndarray:
        k = np.ascontiguousarray(keys).copy()
        rc = self._sort(self._p(k), k.size, dt_of(k), int(descending))
        assert rc == 0, rc
        return k

    def sort_inplace(self, keys: np.ndarray, descending: bool = False) -> None:
        rc = self._sort(self._p(keys), keys.size, dt_of(keys), int(descending))
        assert rc == 0, rc

    def sort_by_key(self, keys: np.ndarray, vals: np.ndarray, descending: bool = False
                    ) -> Tuple[np.ndarray, np.ndarray]:
        k = np.ascontiguousarray(keys).copy()
        v = np.ascontiguousarray(vals).copy()
        self.sort_by_key_inplace(k, v, descending)
        return k, v

    def sort_by_key_inplace(self, k: np.ndarray, v: np.ndarray, descending: bool = False) -> None:
        rc = self._sbk(self._p(k), self._p(v), k.size, dt_of(k), v.dtype.itemsize, int(descending))
        assert rc == 0, rc

    def scan(self, a: np.ndarray, exclusive: bool = False, init=None, inplace: bool = False) -> np.ndarray:
        a = np.ascontiguousarray(a)
        out = a if inplace else np.empty_like(a)
        ini = None if init is None else np.array([init], dtype=a.dtype)
        rc = self._scan(self._p(a), self._p(out), a.size, dt_of(a), int(exclusive), self._p(ini))
        assert rc == 0, rc
        return out

    def scan_by_key(self, keys: np.ndarray, vals: np.ndarray, exclusive: bool = False, init=None) -> np.ndarray:
        keys = np.ascontiguousarray(keys)
        vals = np.ascontiguousarray(vals)
        out = np.empty_like(vals)
        ini = None if init is None else np.array([init], dtype=vals.dtype)
        rc = self._sbk_scan(self._p(keys), self._p(vals), self._p(out), keys.size, dt_of(keys), dt_of(vals),
                            int(exclusive), self._p(ini))
        assert rc == 0, rc
        return out

    def reduce(self, a: np.ndarray, init=None):
        """init + sum of ``a`` in a's type (a numpy scalar of that type)."""
        a = np.ascontiguousarray(a)
        out = np.zeros(1, dtype=a.dtype)
        ini = None if init is None else np.array([init], dtype=a.dtype)
        rc = self._reduce(self._p(a), a.size, dt_of(a), self._p(ini), self._p(out))
        assert rc == 0, rc
        return out[0]

    def reduce_by_key(self, keys: np.ndarray, vals: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
        keys = np.ascontiguousarray(keys)
        vals = np.ascontiguousarray(vals)
        ko = np.empty_like(keys)
        vo = np.empty_like(vals)
        r = self._rbk(self._p(keys), self._p(vals), self._p(ko), self._p(vo), keys.size, dt_of(keys), dt_of(vals))
        assert r >= 0, r
        return ko[:r].copy(), vo[:r].copy()

    def unique_by_key(self, keys: np.ndarray, vals: Optional[np.ndarray] = None, inplace: bool = False
                      ) -> Tuple[np.ndarray, Optional[np.ndarray]]:
        """First (key, value) of every run of equal consecutive keys; vals=None is thrust::unique.
        inplace=True runs the in-place form on copies of the inputs."""
        keys = np.ascontiguousarray(keys)
        vb = 0 if vals is None else vals.dtype.itemsize
        if inplace:
            ko = keys.copy()
            vo = None if vals is None else np.ascontiguousarray(vals).copy()
            r = self._ubk(self._p(ko), self._p(vo), self._p(ko), self._p(vo), keys.size, dt_of(keys), vb)
        else:
            ko = np.empty_like(keys)
            vo = None if vals is None else np.empty_like(vals)
            vin = None if vals is None else np.ascontiguousarray(vals)
            r = self._ubk(self._p(keys), self._p(vin), self._p(ko), self._p(vo), keys.size, dt_of(keys), vb)
        assert r >= 0, r
        return ko[:r].copy(), (None if vo is None else vo[:r].copy())

    def copy_flagged(self, data: np.ndarray, flags: np.ndarray) -> np.ndarray:
        """thrust::copy_if(data, stencil=flags, identity): the elements whose flag is non-zero."""
        data = np.ascontiguousarray(data)
        flags = np.ascontiguousarray(flags)
        out = np.empty_like(data)
        r = self._cpf(self._p(data), self._p(flags), self._p(out), data.size, data.dtype.itemsize, dt_of(flags))
        assert r >= 0, r
        return out[:r].copy()

    def histogram(self, data: np.ndarray, bin_values: np.ndarray) -> np.ndarray:
        d = np.ascontiguousarray(data).copy()
        b = np.ascontiguousarray(bin_values, dtype=d.dtype)
        counts = np.empty(b.size, dtype=np.uint32)
        rc = self._hist(self._p(d), d.size, dt_of(d), self._p(b), b.size, self._p(counts))
        assert rc == 0, rc
        return counts


_cache = {}


def port() -> CpuChecker:
    if "port" not in _cache:
        _cache["port"] = CpuChecker(HERE / "liboracle.so", "oracle_", "port")
    return _cache["port"]


def ref(system: str = "cpp") -> CpuChecker:
    key = "ref_" + system
    if key not in _cache:
        _cache[key] = CpuChecker(HERE / "_ref" / f"libthrust_ref_{system}.so", "ref_", "reference")
    return _cache[key]


def have_ref(system: str = "cpp") -> bool:
    return (HERE / "_ref" / f"libthrust_ref_{system}.so").exists()
