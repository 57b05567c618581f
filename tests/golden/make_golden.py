"""Regenerates tests/golden/reference_vectors.npz from the UNMODIFIED reference.

Run where the reference tree exists (after `make -C oracle ref`):
    python tests/golden/make_golden.py
Every output array is produced by the reference's own CPP device system
(oracle/_ref/libthrust_ref_cpp.so: Thrust 2.2.0 headers compiled in place) on small
seeded inputs; inputs are stored next to the outputs so the fixture does not depend on
a random-number implementation. The file is a few hundred KB and travels with the repo,
so the GPU box can check both the oracle and the CUDA path against reference outputs
without the reference tree.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402

TYPES = ["int8", "uint8", "int16", "uint16", "int32", "uint32", "int64", "uint64", "float32", "float64", "bool"]
NUMERIC = ["int32", "uint32", "int64", "uint64", "float32", "float64"]
N = 1031


def keys_for(rng, name, n):
    dt = np.dtype(name)
    if name == "bool":
        return rng.integers(0, 2, size=n).astype(np.bool_)
    u = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[dt.itemsize]
    raw = rng.integers(0, np.iinfo(u).max, size=n, dtype=u, endpoint=True)
    if dt.kind == "f":  # random bit patterns: NaNs, infinities, subnormals, both zeros; plus duplicates
        raw[: n // 4] = raw[n // 4: 2 * (n // 4)]
        raw[:4] = np.array([0, 1 << (8 * dt.itemsize - 1), 0, 1 << (8 * dt.itemsize - 1)], dtype=u)
    elif dt.itemsize >= 4:
        raw &= u(0xFFFFF)  # duplicates, so that stability shows in the values
    return raw.view(dt)


def main():
    ref = oracle.ref("cpp")
    rng = np.random.default_rng(20240607)
    out = {}
    for t in TYPES:
        k = keys_for(rng, t, N)
        v = rng.integers(0, 1 << 32, size=N, dtype=np.uint32)
        out[f"sort/{t}/keys"] = k
        out[f"sort/{t}/vals"] = v
        for desc in (0, 1):
            out[f"sort/{t}/desc{desc}/keys_only"] = ref.sort(k, bool(desc))
            sk, sv = ref.sort_by_key(k, v, bool(desc))
            out[f"sort/{t}/desc{desc}/by_key_keys"] = sk
            out[f"sort/{t}/desc{desc}/by_key_vals"] = sv
    for t in NUMERIC:
        dt = np.dtype(t)
        a = rng.uniform(-1, 1, size=N).astype(dt) if dt.kind == "f" else \
            rng.integers(np.iinfo(dt).min, np.iinfo(dt).max, size=N, dtype=dt, endpoint=True)
        out[f"scan/{t}/in"] = a
        out[f"scan/{t}/inclusive"] = ref.scan(a)
        out[f"scan/{t}/exclusive"] = ref.scan(a, True)
        out[f"scan/{t}/exclusive_init11"] = ref.scan(a, True, 11)
        keys = np.cumsum(rng.random(N) < 0.3).astype(np.int32)
        vals = rng.uniform(-50, 50, size=N).astype(dt) if dt.kind == "f" else rng.integers(0, 1000, size=N).astype(dt)
        ko, vo = ref.reduce_by_key(keys, vals)
        out[f"rbk/{t}/keys"], out[f"rbk/{t}/vals"] = keys, vals
        out[f"rbk/{t}/out_keys"], out[f"rbk/{t}/out_vals"] = ko, vo
    data = rng.integers(0, 64, size=N).astype(np.int32)
    out["hist/data"] = data
    out["hist/bins"] = np.arange(64, dtype=np.int32)
    out["hist/counts"] = ref.histogram(data, np.arange(64, dtype=np.int32))
    # reduce: drawn last, so the arrays above do not change when this block is extended
    for t in TYPES:
        if t == "bool":
            continue
        dt = np.dtype(t)
        a = rng.uniform(-1, 1, size=N).astype(dt) if dt.kind == "f" else \
            rng.integers(np.iinfo(dt).min, np.iinfo(dt).max, size=N, dtype=dt, endpoint=True)
        out[f"reduce/{t}/in"] = a
        out[f"reduce/{t}/sum"] = np.array([ref.reduce(a)])
        out[f"reduce/{t}/sum_init13"] = np.array([ref.reduce(a, 13)])
    # scan_by_key: drawn after everything above
    for t in NUMERIC:
        dt = np.dtype(t)
        keys = np.cumsum(rng.random(N) < 0.3).astype(np.int32)
        vals = rng.uniform(-50, 50, size=N).astype(dt) if dt.kind == "f" else rng.integers(0, 1000, size=N).astype(dt)
        out[f"sbk/{t}/keys"], out[f"sbk/{t}/vals"] = keys, vals
        out[f"sbk/{t}/inclusive"] = ref.scan_by_key(keys, vals)
        out[f"sbk/{t}/exclusive"] = ref.scan_by_key(keys, vals, True)
        out[f"sbk/{t}/exclusive_init11"] = ref.scan_by_key(keys, vals, True, 11)
    # unique_by_key / unique / copy_if with a stencil: drawn after everything above
    for t in TYPES:
        dt = np.dtype(t)
        ids = np.cumsum(rng.random(N) < 0.3)
        keys = (ids % 2).astype(dt) if dt.itemsize == 1 else ids.astype(dt)
        vals = rng.integers(0, 1 << 32, size=N, dtype=np.uint32)
        out[f"ubk/{t}/keys"], out[f"ubk/{t}/vals"] = keys, vals
        out[f"ubk/{t}/out_keys"], out[f"ubk/{t}/out_vals"] = ref.unique_by_key(keys, vals)
        ik, iv = ref.unique_by_key(keys, vals, inplace=True)
        assert ik.tobytes() == out[f"ubk/{t}/out_keys"].tobytes() and iv.tobytes() == out[f"ubk/{t}/out_vals"].tobytes()
        out[f"ubk/{t}/unique"] = ref.unique_by_key(keys)[0]
        flags = (rng.random(N) < 0.4).astype(dt)
        out[f"cpf/{t}/flags"] = flags
        out[f"cpf/{t}/out"] = ref.copy_flagged(vals, flags)
    np.savez_compressed(Path(__file__).with_name("reference_vectors.npz"), **out)
    print("wrote", len(out), "arrays; reference Thrust version", ref.thrust_version)


if __name__ == "__main__":
    main()
