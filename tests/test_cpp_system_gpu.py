"""Runs the C++ boundary test: thrust:: algorithms through thrust_b200::system
(include/thrust_b200/system.h) over the C ABI, compared with Thrust's host system."""
import subprocess
from pathlib import Path

import pytest

BIN = Path(__file__).resolve().parent / "cpp" / "bin" / "test_system"


@pytest.mark.gpu
def test_thrust_custom_system_boundary():
    assert BIN.exists(), "tests/cpp/bin/test_system missing: run __graft_entry__.build()"
    r = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:], r.stderr[-3000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PASSED" in r.stdout


@pytest.mark.gpu
def test_sample_sort_entry_point_from_cpp():
    exe = BIN.parent / "test_sample_sort"
    assert exe.exists(), "tests/cpp/bin/test_sample_sort missing: run __graft_entry__.build()"
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(r.stdout[-2000:], r.stderr[-2000:])
    assert r.returncode == 0 and "PASSED" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
