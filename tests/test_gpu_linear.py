"""The fully connected layer with bias and activation in the GEMM's epilogue (nb2_linear_bias_act_fwd, tcgen05
tensor cores, bf16) through the C ABI: against the reference's own FC layer (golden), the fp64 oracle and, at the
feed-forward sizes of the transformer blocks, sampled rows of the oracle plus linearity in the bias."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import bits, check, to_dev
from thot_b200 import abi

pytestmark = pytest.mark.gpu


def test_golden_reference_fc_layer(golden_dir):
    z = np.load(golden_dir / "fc_act.npz")
    x, w, b = (to_dev(z[k], torch.bfloat16) for k in ("x", "weight", "bias"))
    for name, code in (("none", abi.ACT_NONE), ("gelu", abi.ACT_GELU), ("silu", abi.ACT_SILU)):
        y, pre = abi.linear_bias_act_fwd(x, w, b, code, want_z=True)
        check(y, z[f"{name}_y_f64"], f"y {name}")
        check(pre, z["z_f64"], "pre-activation")
        y2, none = abi.linear_bias_act_fwd(x, w, b, code)
        assert none is None and torch.equal(y, y2)                     # the same epilogue with and without the second output
    y, _ = abi.linear_bias_act_fwd(x, w, None, abi.ACT_GELU)
    check(y, z["nobias_gelu_y_f64"], "y without bias")


@pytest.mark.parametrize("act", [abi.ACT_NONE, abi.ACT_GELU, abi.ACT_SILU])
@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (5, 24, 40), (128, 128, 64), (129, 136, 72), (300, 1024, 256), (1000, 768, 3072), (77, 3072, 768)])
def test_against_oracle(act, M, N, K):
    gen = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=gen).bfloat16(); w = (torch.randn(N, K, generator=gen) / K ** 0.5).bfloat16()
    b = (0.1 * torch.randn(N, generator=gen)).bfloat16()
    ref = O.linear_act(x.float().numpy(), w.float().numpy(), b.float().numpy(), act)
    y, pre = abi.linear_bias_act_fwd(x.cuda(), w.cuda(), b.cuda(), act, want_z=True)
    check(pre, ref["z"], "z")
    check(y, ref["y"], "y")
    assert abi.device_status() == 0


def test_feed_forward_size_sampled_rows_and_bias_linearity():
    """[16384, 1024] x [4096, 1024]^T, the up-projection of a transformer block's feed forward: rows sampled against
    the oracle; with the identity epilogue, adding a constant to the bias adds it to every output (before rounding)."""
    M, N, K = 16384, 4096, 1024
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(M, K, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=gen) / 32).bfloat16()
    b = (0.1 * torch.randn(N, device="cuda", generator=gen)).bfloat16()
    y, _ = abi.linear_bias_act_fwd(x, w, b, abi.ACT_GELU)
    idx = torch.linspace(0, M - 1, 40).long().cuda()
    ref = O.linear_act(x[idx].float().cpu().numpy(), w.float().cpu().numpy(), b.float().cpu().numpy(), O.ACT_GELU)
    check(y[idx], ref["y"], "sampled rows")
    assert torch.equal(y, abi.linear_bias_act_fwd(x, w, b, abi.ACT_GELU)[0])           # deterministic
    z0, _ = abi.linear_bias_act_fwd(x, w, None, abi.ACT_NONE)
    z1, _ = abi.linear_bias_act_fwd(x, w, torch.full((N,), 2.0, device="cuda").bfloat16(), abi.ACT_NONE)
    tol.bf16_ulp_close(bits(z1[idx]), z0[idx].float().cpu().numpy().astype(np.float64) + 2.0, max_ulp=1)


def test_argument_checks():
    L = abi.lib()
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 4, 8, 8, abi.F32, 0, None, 0, None) == -3      # fp32 is not taken
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 4, 12, 8, abi.BF16, 0, None, 0, None) == -2    # N % 8
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 0, 8, 8, abi.BF16, 0, None, 0, None) == 0      # empty
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 4, 8, 8, abi.BF16, 0, None, 0, None) == -1     # NULL
