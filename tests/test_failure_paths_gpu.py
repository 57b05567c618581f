"""Failure paths on the GPU without faulting it: a wait that runs out must come back as a
status code, and the device must stay usable afterwards."""
import numpy as np
import pytest
import torch

import thrust_b200 as tb
from thrust_b200 import _capi as capi

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_survives(cuda_device):
    rc = capi.lib.tb200_selftest_wait_timeout(2000, None)
    assert rc == capi.ERR_WAIT_TIMEOUT
    assert "wait" in capi.error_string(rc)
    # the context is intact: a real algorithm runs and is correct
    x = torch.arange(100000, dtype=torch.int64, device=cuda_device)
    y = tb.inclusive_scan(x)
    assert int(y[-1]) == 99999 * 100000 // 2
    assert torch.cuda.is_available() and torch.zeros(1, device=cuda_device).item() == 0.0


def test_python_front_end_raises_on_device_status(cuda_device):
    with pytest.raises(tb.Tb200Error) as e:
        capi.check(capi.lib.tb200_selftest_wait_timeout(100, None), "selftest")
    assert e.value.code == capi.ERR_WAIT_TIMEOUT
