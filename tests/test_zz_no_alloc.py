"""nb2_layernorm_bwd_static: the backward for hosts that may not allocate device memory
(its partials scratch is a fixed array inside the library).  Collected last on purpose: it
shares one device array between calls, and a failure here must not hide the other tests.

Checked through the C ABI against the ordinary entry points (nb2_layernorm_bwd +
nb2_colreduce_partials with a caller-allocated workspace) and against the CPU oracle, on two
calls in a row.  "Allocates nothing" is checked with the driver's own count of free device
memory (cudaMemGetInfo through torch.cuda.mem_get_info), which sees every allocation of the
process whoever makes it, not only the ones that go through torch's caching allocator."""
from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import check, make
from thot_b200 import abi

pytestmark = pytest.mark.gpu


def _static_bwd(x, dy, gamma, beta, mean, rstd, act, dx, grads):
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rows, D = x.shape
    return abi.lib().nb2_layernorm_bwd_static(P(x), P(dy), P(gamma), P(beta), P(mean), P(rstd), P(dx), P(grads), rows, D,
                                              abi.dtype_code(x.dtype), act, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype,D", [(torch.float32, 1024), (torch.bfloat16, 2048), (torch.float32, 513)])
def test_static_scratch_backward_matches_the_allocating_path_twice(dtype, D):
    rows = 3000
    act = abi.ACT_GELU
    for call in range(2):                               # the second call reuses the array with stale contents
        x, xn = make((rows, D), 100 + call, dtype)
        dy, dyn = make((rows, D), 200 + call, dtype)
        gamma, gn = make((D,), 300 + call, dtype, 0.02, 1.0)
        beta, bn = make((D,), 400 + call, dtype, 0.02)
        y, mean, rstd = abi.layernorm_fwd(x, gamma, beta, 1e-5, act)
        dx_ref, grads_ref = abi.layernorm_bwd(x, dy, gamma, beta, mean, rstd, act)
        dx = torch.empty_like(x)
        grads = torch.full((2, D), float("nan"), device="cuda")
        if call == 0:
            # the first call on a device also looks up the array's address; make it before measuring
            assert _static_bwd(x, dy, gamma, beta, mean, rstd, act, dx, grads) == 0
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        assert _static_bwd(x, dy, gamma, beta, mean, rstd, act, dx, grads) == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, (free_before, free_after)       # no cudaMalloc by anybody during the call
        assert torch.cuda.memory_allocated() <= torch_before
        assert torch.equal(dx, dx_ref)                                      # same kernel, same grid: identical
        assert torch.equal(grads, grads_ref)
        ref = O.layernorm_act(xn, gn, bn, dyn, 1e-5, act)                   # and against the oracle directly
        check(dx, ref["dx"], "dx")
        tol.long_sum_close(grads[0].cpu().numpy(), ref["dgamma"], rows)
        tol.long_sum_close(grads[1].cpu().numpy(), ref["dbeta"], rows)
    assert abi.device_status() == 0


def test_static_scratch_backward_limits_and_empty_batch():
    D = 8192                                            # 148 partials x 2 x 8192 floats exceed the built-in array
    x, _ = make((4096, D), 1, torch.float32)
    g, _ = make((D,), 2, torch.float32, 0.02, 1.0)
    b, _ = make((D,), 3, torch.float32, 0.02)
    y, mean, rstd = abi.layernorm_fwd(x, g, b, 1e-5, 0)
    dx = torch.empty_like(x)
    grads = torch.zeros(2, D, device="cuda")
    assert _static_bwd(x, x, g, b, mean, rstd, 0, dx, grads) == -5
    assert b"built-in array" in abi.lib().nb2_last_error_string()
    e = torch.empty(0, 256, device="cuda")
    grads = torch.ones(2, 256, device="cuda")
    assert _static_bwd(e, e, g[:256].contiguous(), b[:256].contiguous(), mean[:0], rstd[:0], 0, e, grads) == 0
    torch.cuda.synchronize()
    assert float(grads.abs().sum()) == 0.0
