"""tb200_scan_static — the scan entry point that allocates nothing (its look-back scratch is a
fixed array inside the library) — must give exactly what tb200_scan gives, on two calls in a
row (the second call finds the first call's descriptors in the shared array and has to clear
them itself), and what the CPU oracle gives. Collected last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from thrust_b200 import _capi as capi

pytestmark = pytest.mark.gpu


def _scan(entry, x: torch.Tensor, dtype: int, exclusive: int, init) -> torch.Tensor:
    out = torch.empty_like(x)
    stream = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    n = x.numel()
    if entry == "static":
        rc = capi.lib.tb200_scan_static(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), n, dtype, exclusive,
                                        init, stream)
        capi.check(rc, "tb200_scan_static")
        # the device status word of the library's own array (a bounded wait that ran out would show here)
        capi.check(capi.lib.tb200_scan_static_status(stream), "tb200_scan_static_status")
    else:
        need = C.c_size_t(0)
        capi.check(capi.lib.tb200_scan(None, C.byref(need), None, None, n, dtype, exclusive, init, stream), "size")
        temp = torch.empty(need.value, dtype=torch.uint8, device=x.device)
        capi.check(capi.lib.tb200_scan(C.c_void_p(temp.data_ptr()), C.byref(need), C.c_void_p(x.data_ptr()),
                                       C.c_void_p(out.data_ptr()), n, dtype, exclusive, init, stream), "tb200_scan")
        capi.check(capi.lib.tb200_temp_status(C.c_void_p(temp.data_ptr()), stream), "status")
    torch.cuda.synchronize(x.device)
    return out


def test_static_scan_matches_scan_twice_in_a_row(cuda_device):
    rng = np.random.default_rng(99)
    cases = [
        (capi.I64, torch.from_numpy(rng.integers(-(1 << 40), 1 << 40, size=(1 << 21) + 12345)), 0, None),
        (capi.I32, torch.from_numpy(rng.integers(-1000, 1000, size=300001).astype(np.int32)), 1, C.byref(C.c_int32(7))),
        (capi.F32, torch.from_numpy(rng.uniform(-1, 1, size=(1 << 20) + 3).astype(np.float32)), 0, None),
        (capi.F64, torch.from_numpy(rng.uniform(-1, 1, size=70001)), 1, C.byref(C.c_double(0.25))),
    ]
    for call in range(2):  # the second round reuses a dirty scratch array
        for dtype, host, exclusive, init in cases:
            x = host.to(cuda_device)
            want = _scan("plain", x, dtype, exclusive, init)
            got = _scan("static", x, dtype, exclusive, init)
            ini = None if init is None else init._obj.value
            cpu = torch.from_numpy(oracle.port().scan(host.numpy(), bool(exclusive), ini))
            if dtype in (capi.F32, capi.F64):
                tol = 1e-5 * float(host.abs().double().sum())
                assert float((got.double() - want.double()).abs().max()) <= tol, (call, dtype)
                assert float((got.cpu().double() - cpu.double()).abs().max()) <= tol, (call, dtype)
            else:
                assert torch.equal(got, want), (call, dtype)
                assert torch.equal(got.cpu(), cpu), (call, dtype)


def test_static_scan_limits_are_the_documented_ones(cuda_device):
    # Size path only: with NULL data pointers nothing is launched. At the documented maximum the
    # call gets as far as the argument check; one element more is refused as an overflow.
    for dtype, limit in ((capi.F32, 1 << 31), (capi.I32, 1 << 31), (capi.I64, 1 << 29), (capi.F64, 1 << 29)):
        assert capi.lib.tb200_scan_static(None, None, limit, dtype, 0, None, None) == capi.ERR_INVALID_ARGUMENT
        assert capi.lib.tb200_scan_static(None, None, limit + 1, dtype, 0, None, None) == capi.ERR_OVERFLOW
    assert capi.lib.tb200_scan_static(None, None, (1 << 31) + (1 << 20), capi.I64, 0, None, None) == capi.ERR_OVERFLOW
    assert capi.lib.tb200_scan_static(None, None, 0, capi.I16, 0, None, None) == capi.ERR_UNSUPPORTED
    torch.cuda.synchronize(cuda_device)
    assert capi.lib.tb200_scan_static_status(None) == 0
