"""Parity of the sort-based dense histogram (tb200_radix_sort + tb200_histogram_sorted through the
C ABI) with the CPU oracle.

The recipe is the reference's examples/histogram.cu:60-101: sort a copy of the data, take the
upper bound of every bin value (cumulative counts), then the difference of neighbours. Counts
are integers, so every comparison is exact. The known answer is the example's own output
(internal/test/thrust.example.histogram.filecheck); the committed reference vectors come from
the reference's CPU system.
"""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
import thrust_b200 as tb
from util import to_device, to_host

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
DTYPES = [np.int32, np.uint32, np.int64, np.uint64, np.float32, np.float64]
# 8192 and 10240 are tile sizes of the sort's passes; 300007 spans many tiles
SIZES = [0, 1, 2, 255, 256, 257, 8191, 8192, 8193, 10239, 10240, 10241, 300007]


def _data(rng, n, dtype, span):
    """n draws from `span` distinct values around zero (negative ones too where the type has them)."""
    lo = 0 if np.dtype(dtype).kind == "u" else -(span // 2)
    return rng.integers(lo, lo + span, size=n).astype(dtype)


def _both(data, bins):
    """(counts from histogram_sorted on data sorted by the library, counts from dense_histogram)."""
    d = to_device(data)
    b = to_device(bins)
    work = d.clone()
    tb.sort(work)
    split = to_host(tb.histogram_sorted(work, b), np.uint32)
    whole = to_host(tb.dense_histogram(d, b), np.uint32)
    assert to_host(d, data.dtype).tobytes() == data.tobytes()  # dense_histogram works on a copy
    return split, whole


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_histogram_matches_oracle(cuda_device, n, dtype):
    rng = np.random.default_rng(500 + n)
    chk = oracle.port()
    for num_bins in (1, 9, 300):
        data = _data(rng, n, dtype, num_bins + 3)  # some values fall outside every bin
        lo = 0 if np.dtype(dtype).kind == "u" else -(num_bins // 2)
        bins = np.arange(lo, lo + num_bins).astype(dtype)
        want = chk.histogram(data, bins)
        split, whole = _both(data, bins)
        assert split.tolist() == want.tolist(), (num_bins, "histogram_sorted")
        assert whole.tolist() == want.tolist(), (num_bins, "dense_histogram")


@pytest.mark.parametrize("dtype", [np.int32, np.float32])
def test_histogram_65536_bins(cuda_device, dtype):
    # the bin count of the benchmark configuration, skewed towards small values
    rng = np.random.default_rng(65536)
    n = 1_000_003
    data = np.minimum(rng.zipf(1.2, size=n), 65535).astype(dtype)
    bins = np.arange(65536).astype(dtype)
    want = oracle.port().histogram(data, bins)
    split, whole = _both(data, bins)
    assert split.tolist() == want.tolist()
    assert whole.tolist() == want.tolist()
    assert int(want.astype(np.int64).sum()) == n


def test_histogram_duplicate_bin_values(cuda_device):
    # a repeated bin value takes everything on its first occurrence and nothing afterwards
    data = np.array([5, 1, 3, 3, 7, 3, 1, 9], dtype=np.int32)
    bins = np.array([1, 3, 3, 3, 8, 8, 9], dtype=np.int32)
    want = oracle.port().histogram(data, bins)
    split, whole = _both(data, bins)
    assert want.tolist() == [2, 3, 0, 0, 2, 0, 1]
    assert split.tolist() == want.tolist() and whole.tolist() == want.tolist()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_histogram_signed_zeros_share_a_bin(cuda_device, dtype):
    # the sort orders -0.0 before +0.0 (bitwise order), the search compares with operator<,
    # under which the two are equal: both are counted in the bin whose value is zero
    data = np.array([0.0, -0.0, -1.0, 0.0, 2.5, -0.0, -0.0, 1.0], dtype=dtype)
    for zero in (0.0, -0.0):
        bins = np.array([-1.0, zero, 1.0, 3.0], dtype=dtype)
        want = oracle.port().histogram(data, bins)
        split, whole = _both(data, bins)
        assert want.tolist() == [1, 5, 1, 1]
        assert split.tolist() == want.tolist() and whole.tolist() == want.tolist()


def test_histogram_example_known_answer(cuda_device):
    # examples/histogram.cu:21-25 with the expected output of internal/test/thrust.example.histogram.filecheck
    s = json.loads((GOLDEN / "known_answers.json").read_text())["dense_histogram_example"]
    data = np.array(s["data"], dtype=np.int32)
    bins = np.arange(len(s["histogram"]), dtype=np.int32)
    d = to_device(data)
    work = d.clone()
    tb.sort(work)
    assert to_host(work, np.int32).tolist() == s["sorted"]
    split, whole = _both(data, bins)
    assert split.tolist() == s["histogram"] and whole.tolist() == s["histogram"]
    assert np.cumsum(split).tolist() == s["cumulative"]


def test_histogram_matches_reference_vectors(cuda_device):
    z = np.load(GOLDEN / "reference_vectors.npz")
    data, bins = z["hist/data"], z["hist/bins"]
    split, whole = _both(data, bins.astype(data.dtype))
    assert split.tolist() == z["hist/counts"].tolist()
    assert whole.tolist() == z["hist/counts"].tolist()


def test_histogram_sorted_with_no_bins_or_no_data(cuda_device):
    empty = torch.empty(0, dtype=torch.int32, device=cuda_device)
    some = to_device(np.array([1, 2, 3], dtype=np.int32))
    assert tb.histogram_sorted(some, empty).numel() == 0
    assert to_host(tb.histogram_sorted(empty, some), np.uint32).tolist() == [0, 0, 0]
