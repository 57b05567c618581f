"""Pins the CPU oracle (oracle/oracle.c): against the reference's known-answer vectors,
against outputs of the unmodified reference committed as tests/golden/reference_vectors.npz,
and — where oracle/_ref is built — against the reference's CPP and OMP systems live."""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLD = Path(__file__).resolve().parent / "golden"
KA = json.loads((GOLD / "known_answers.json").read_text())
TYPES = ["int8", "uint8", "int16", "uint16", "int32", "uint32", "int64", "uint64", "float32", "float64", "bool"]
NUMERIC = ["int32", "uint32", "int64", "uint64", "float32", "float64"]


@pytest.fixture(scope="module")
def port():
    oracle.build(ref=False)
    return oracle.port()


@pytest.fixture(scope="module")
def vectors():
    return np.load(GOLD / "reference_vectors.npz")


def test_known_answers(port):
    s = KA["sort_simple"]
    assert port.sort(np.array(s["keys"], dtype=np.int32)).tolist() == s["sorted"]
    s = KA["sort_by_key_simple"]
    k, v = port.sort_by_key(np.array(s["keys"], dtype=np.int32), np.array(s["values"], dtype=np.int32))
    assert k.tolist() == s["sorted_keys"] and v.tolist() == s["sorted_values"]
    s = KA["scan_simple"]
    a = np.array(s["input"], dtype=np.int32)
    assert port.scan(a).tolist() == s["inclusive"]
    assert port.scan(a, True).tolist() == s["exclusive"]
    assert port.scan(a, True, 3).tolist() == s["exclusive_init_3"]
    assert port.scan(a.copy(), inplace=True).tolist() == s["inclusive"]
    s = KA["scan_mixed_types"]
    f = np.array(s["float_input"], dtype=np.float32)
    assert port.scan(f).tolist() == s["float_inclusive"]
    assert port.scan(f, True, 5.5).tolist() == s["float_exclusive_init_5.5"]
    assert port.scan(np.array(s["int_input"], dtype=np.int32)).tolist() == s["int_inclusive"]
    s = KA["reduce_simple"]
    for dt in (np.int8, np.int32, np.int64, np.float32, np.float64):
        a = np.array(s["input"], dtype=dt)
        assert port.reduce(a) == s["sum"] and port.reduce(a, 10) == s["sum_init_10"]
    s = KA["scan_by_key_simple"]
    for kd in (np.int8, np.int32, np.uint64, np.float32):
        k, v = np.array(s["keys"], dtype=kd), np.array(s["values"], dtype=np.int32)
        assert port.scan_by_key(k, v).tolist() == s["inclusive"]
        assert port.scan_by_key(k, v, True).tolist() == s["exclusive"]
        assert port.scan_by_key(k, v, True, 10).tolist() == s["exclusive_init_10"]
    s = KA["reduce_by_key_simple"]
    for dt in (np.int8, np.int32, np.uint64):
        ko, vo = port.reduce_by_key(np.array(s["keys"], dtype=dt), np.array(s["values"], dtype=np.int32))
        assert ko.tolist() == s["out_keys"] and vo.tolist() == s["out_values"]
    s = KA["unique_by_key_simple"]
    for dt in (np.int8, np.int32, np.uint64, np.float32):
        k, v = np.array(s["keys"], dtype=dt), np.array(s["values"], dtype=np.int32)
        for inplace in (False, True):
            ko, vo = port.unique_by_key(k, v, inplace)
            assert ko.tolist() == s["out_keys"] and vo.tolist() == s["out_values"]
        assert port.unique_by_key(k)[0].tolist() == s["out_keys"]
    s = KA["dense_histogram_example"]
    data = np.array(s["data"], dtype=np.int32)
    assert port.sort(data).tolist() == s["sorted"]
    assert port.histogram(data, np.arange(9, dtype=np.int32)).tolist() == s["histogram"]
    assert np.cumsum(s["histogram"]).tolist() == s["cumulative"]


@pytest.mark.parametrize("t", TYPES)
def test_sort_matches_reference_vectors(port, vectors, t):
    k, v = vectors[f"sort/{t}/keys"], vectors[f"sort/{t}/vals"]
    for desc in (0, 1):
        assert port.sort(k, bool(desc)).tobytes() == vectors[f"sort/{t}/desc{desc}/keys_only"].tobytes()
        sk, sv = port.sort_by_key(k, v, bool(desc))
        assert sk.tobytes() == vectors[f"sort/{t}/desc{desc}/by_key_keys"].tobytes()
        assert sv.tobytes() == vectors[f"sort/{t}/desc{desc}/by_key_vals"].tobytes()


@pytest.mark.parametrize("t", NUMERIC)
def test_scan_and_rbk_match_reference_vectors(port, vectors, t):
    a = vectors[f"scan/{t}/in"]
    assert port.scan(a).tobytes() == vectors[f"scan/{t}/inclusive"].tobytes()
    assert port.scan(a, True).tobytes() == vectors[f"scan/{t}/exclusive"].tobytes()
    assert port.scan(a, True, 11).tobytes() == vectors[f"scan/{t}/exclusive_init11"].tobytes()
    ko, vo = port.reduce_by_key(vectors[f"rbk/{t}/keys"], vectors[f"rbk/{t}/vals"])
    assert ko.tobytes() == vectors[f"rbk/{t}/out_keys"].tobytes()
    assert vo.tobytes() == vectors[f"rbk/{t}/out_vals"].tobytes()


@pytest.mark.parametrize("t", [t for t in TYPES if t != "bool"])
def test_reduce_matches_reference_vectors(port, vectors, t):
    a = vectors[f"reduce/{t}/in"]
    assert np.array([port.reduce(a)]).tobytes() == vectors[f"reduce/{t}/sum"].tobytes()
    assert np.array([port.reduce(a, 13)]).tobytes() == vectors[f"reduce/{t}/sum_init13"].tobytes()


@pytest.mark.parametrize("t", NUMERIC)
def test_scan_by_key_matches_reference_vectors(port, vectors, t):
    k, v = vectors[f"sbk/{t}/keys"], vectors[f"sbk/{t}/vals"]
    assert port.scan_by_key(k, v).tobytes() == vectors[f"sbk/{t}/inclusive"].tobytes()
    assert port.scan_by_key(k, v, True).tobytes() == vectors[f"sbk/{t}/exclusive"].tobytes()
    assert port.scan_by_key(k, v, True, 11).tobytes() == vectors[f"sbk/{t}/exclusive_init11"].tobytes()


@pytest.mark.parametrize("t", TYPES)
def test_unique_by_key_and_copy_flagged_match_reference_vectors(port, vectors, t):
    k, v = vectors[f"ubk/{t}/keys"], vectors[f"ubk/{t}/vals"]
    for inplace in (False, True):
        ko, vo = port.unique_by_key(k, v, inplace)
        assert ko.tobytes() == vectors[f"ubk/{t}/out_keys"].tobytes()
        assert vo.tobytes() == vectors[f"ubk/{t}/out_vals"].tobytes()
    assert port.unique_by_key(k)[0].tobytes() == vectors[f"ubk/{t}/unique"].tobytes()
    assert port.copy_flagged(v, vectors[f"cpf/{t}/flags"]).tobytes() == vectors[f"cpf/{t}/out"].tobytes()


def test_histogram_matches_reference_vectors(port, vectors):
    assert port.histogram(vectors["hist/data"], vectors["hist/bins"]).tolist() == vectors["hist/counts"].tolist()


def test_edge_cases(port):
    for t in TYPES:
        e = np.empty(0, dtype=t)
        assert port.sort(e).size == 0
        one = np.ones(1, dtype=t)
        assert port.sort(one, True).tolist() == one.tolist()
    k, v = port.reduce_by_key(np.empty(0, dtype=np.int32), np.empty(0, dtype=np.float32))
    assert k.size == 0 and v.size == 0
    assert port.reduce(np.empty(0, dtype=np.int32)) == 0 and port.reduce(np.empty(0, dtype=np.float32), 2.5) == 2.5
    # float keys: bitwise total order, -0.0 before +0.0, NaNs at the ends by sign
    f = np.array([0.0, -0.0, np.inf, -np.inf, 1.0, -1.0], dtype=np.float32)
    assert port.sort(f).view(np.uint32).tolist() == np.array([-np.inf, -1.0, -0.0, 0.0, 1.0, np.inf], dtype=np.float32).view(np.uint32).tolist()
    # descending sort_by_key keeps equal keys in input order
    k, v = port.sort_by_key(np.array([1, 2, 1, 2], dtype=np.int16), np.array([0, 1, 2, 3], dtype=np.uint32), True)
    assert k.tolist() == [2, 2, 1, 1] and v.tolist() == [1, 3, 0, 2]


@pytest.mark.skipif(not oracle.have_ref("cpp"), reason="oracle/_ref not built (no reference tree on this machine)")
@pytest.mark.parametrize("system", ["cpp", "omp"])
def test_port_matches_live_reference(port, system):
    if not oracle.have_ref(system):
        pytest.skip(system)
    ref = oracle.ref(system)
    assert ref.thrust_version == 200200
    rng = np.random.default_rng(5)
    for t in TYPES:
        n = 20011
        dt = np.dtype(t)
        if t == "bool":
            k = rng.integers(0, 2, size=n).astype(np.bool_)
        elif dt.kind == "f":
            # finite keys without -0.0: the OMP system's merge step treats -0.0 == +0.0, so its
            # order of mixed zeros depends on the thread count (omp/detail/sort.inl:48-60)
            k = rng.uniform(-1e6, 1e6, size=n).astype(dt)
        else:
            k = rng.integers(np.iinfo(dt).min, np.iinfo(dt).max, size=n, dtype=dt, endpoint=True)
        v = rng.integers(0, 1 << 32, size=n, dtype=np.uint32)
        for desc in (False, True):
            assert port.sort(k, desc).tobytes() == ref.sort(k, desc).tobytes()
            a, b = port.sort_by_key(k, v, desc), ref.sort_by_key(k, v, desc)
            assert a[0].tobytes() == b[0].tobytes() and a[1].tobytes() == b[1].tobytes()
    for t in TYPES:
        dt = np.dtype(t)
        n = 20011
        ids = np.cumsum(rng.random(n) < 0.2)
        keys = (ids % 2).astype(dt) if dt.itemsize == 1 else ids.astype(dt)
        for vd in (None, np.uint8, np.uint16, np.uint32, np.uint64):
            vals = None if vd is None else rng.integers(0, 200, size=n).astype(vd)
            for inplace in (False, True):
                x, y = port.unique_by_key(keys, vals, inplace), ref.unique_by_key(keys, vals, inplace)
                assert x[0].tobytes() == y[0].tobytes()
                assert vals is None or x[1].tobytes() == y[1].tobytes()
            if vals is not None:
                flags = (rng.random(n) < 0.5).astype(dt)
                assert port.copy_flagged(vals, flags).tobytes() == ref.copy_flagged(vals, flags).tobytes()
    for t in NUMERIC:
        dt = np.dtype(t)
        a = rng.uniform(-1, 1, size=30011).astype(dt) if dt.kind == "f" else rng.integers(0, 1000, size=30011).astype(dt)
        for ex, init in [(False, None), (True, None), (True, 7)]:
            assert port.scan(a, ex, init).tobytes() == ref.scan(a, ex, init).tobytes()
        keys = np.cumsum(rng.random(30011) < 0.1).astype(np.int64)
        x, y = port.reduce_by_key(keys, a), ref.reduce_by_key(keys, a)
        assert x[0].tobytes() == y[0].tobytes()
        if dt.kind != "f" or system == "cpp":  # the OMP system reduces through a parallel scan: float order differs
            assert x[1].tobytes() == y[1].tobytes()
        else:
            assert np.allclose(x[1], y[1], rtol=1e-4, atol=1e-3)
        for ex, init in [(False, None), (True, None), (True, 7)]:
            x, y = port.scan_by_key(keys, a, ex, init), ref.scan_by_key(keys, a, ex, init)
            if dt.kind != "f" or system == "cpp":
                assert x.tobytes() == y.tobytes()
            else:
                assert np.allclose(x, y, rtol=1e-4, atol=1e-3)
        for init in (None, 7):
            if dt.kind != "f" or system == "cpp":  # the OMP system adds per-thread partial sums
                assert np.array([port.reduce(a, init)]).tobytes() == np.array([ref.reduce(a, init)]).tobytes()
            else:
                assert abs(float(port.reduce(a, init)) - float(ref.reduce(a, init))) <= 1e-5 * float(np.abs(a).sum())
