"""The host-buffer entry point (nb2_layernorm_act_step_host) against the device-pointer path."""
from __future__ import annotations

import pytest
import torch

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import check
from thot_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,chunk", [(1000, 128), (4096, 0), (77, 1000)])
def test_host_step_matches_device_path(rows, chunk):
    D = 1024
    gen = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, D, generator=gen).pin_memory()
    dy = torch.randn(rows, D, generator=gen).pin_memory()
    gamma = 1 + 0.02 * torch.randn(D, generator=gen)
    beta = 0.02 * torch.randn(D, generator=gen)
    y = torch.empty_like(x).pin_memory()
    dx = torch.empty_like(x).pin_memory()
    gb = torch.empty(2, D).pin_memory()
    hs = abi.HostStep(rows, D, torch.float32, chunk)
    for _ in range(2):                                   # twice: buffer sets are reused
        hs.step(x, dy, gamma, beta, y, dx, gb, 1e-5, abi.ACT_GELU)
    hs.close()
    yd, mean, rstd = abi.layernorm_fwd(x.cuda(), gamma.cuda(), beta.cuda(), 1e-5, abi.ACT_GELU)
    dxd, gbd = abi.layernorm_bwd(x.cuda(), dy.cuda(), gamma.cuda(), beta.cuda(), mean, rstd, abi.ACT_GELU)
    assert torch.equal(y, yd.cpu()) and torch.equal(dx, dxd.cpu())           # same kernels, row-independent
    ref = O.layernorm_act(x.numpy(), gamma.numpy(), beta.numpy(), dy.numpy(), 1e-5, O.ACT_GELU)
    tol.long_sum_close(gb[0].numpy(), ref["dgamma"], rows)
    tol.long_sum_close(gb[1].numpy(), ref["dbeta"], rows)
    tol.fp32_close(gb.numpy(), gbd.cpu().numpy(), rtol=1e-5, atol=1e-5)


def test_host_step_rejects_mismatched_shapes():
    hs = abi.HostStep(64, 256, torch.float32)
    x = torch.zeros(128, 256)
    with pytest.raises(abi.Nb2Error):
        hs.step(x, x, torch.ones(256), torch.zeros(256), x.clone(), x.clone(), torch.zeros(2, 256), 1e-5, 0)
    hs.close()
