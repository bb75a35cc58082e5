"""Failure detection without a GPU fault: a device-side wait that cannot complete must run out of
its (short) limit, leave an error code for the host, and leave the context usable."""
from __future__ import annotations

import ctypes

import pytest
import torch

from tests.gpu_util import make
from thot_b200 import abi

pytestmark = pytest.mark.gpu


def test_wait_on_a_barrier_nothing_completes_times_out_and_reports():
    assert abi.device_status() == 0
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    limit = 2_000_000                                   # about a millisecond of SM cycles
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    abi.check(abi.lib().nb2_selftest_bounded_wait(limit, ctypes.c_void_p(waited.data_ptr()), st))
    torch.cuda.synchronize()                            # returns: the kernel ended by itself
    assert limit <= int(waited.item()) < 100 * limit    # it waited the limit, not forever
    with pytest.raises(abi.Nb2Error) as err:
        abi.device_status()
    assert err.value.status == -6 and "code 3" in str(err.value)
    assert abi.device_status() == 0                     # reading cleared the word
    # the context is intact: an ordinary call works and reports nothing
    x, _ = make((512, 1024), 1, torch.float32)
    g, _ = make((1024,), 2, torch.float32, 0.02, 1.0)
    b, _ = make((1024,), 3, torch.float32, 0.02)
    y, mean, rstd = abi.layernorm_fwd(x, g, b, 1e-5, abi.ACT_GELU)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all() and abi.device_status() == 0


def test_selftest_rejects_unbounded_limits():
    assert abi.lib().nb2_selftest_bounded_wait(0, None, None) == -2
    assert abi.lib().nb2_selftest_bounded_wait(10**12, None, None) == -2
