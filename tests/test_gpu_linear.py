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

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not abi.linear_available(), reason="libnott_b200_linear.so is not installed next to the core library")]


def gemm_check(got, ref, x, w, b, what):
    """bf16 outputs of a K-term fp32-accumulated dot product: within 2 bf16 ulp of the fp64 result, or -- where the
    terms cancel -- inside the accumulation's own error bound 4 u sum_k |x_k w_k| (u = 2^-24), the GEMM counterpart
    of the absolute floor the row kernels' checks use."""
    bound = 2.0 ** -22 * (np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64).T + (0 if b is None else np.abs(b)))
    ok = tol.bf16_ulp_mask(bits(got), ref) | (np.abs(got.float().cpu().numpy().astype(np.float64) - ref) <= bound)
    assert ok.all(), f"{what}: {(~ok).sum()} of {ok.size} elements outside 2 bf16 ulp and the accumulation bound"


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
    xn, wn, bn = x.float().numpy(), w.float().numpy(), b.float().numpy()
    gemm_check(pre, ref["z"], xn, wn, bn, "z")
    gemm_check(y, ref["y"], xn, wn, bn, "y")             # |act'| <= 1.13, so the same bound carries over
    assert abi.device_status() == 0


def test_feed_forward_size_sampled_rows_and_bias_as_a_column():
    """[16384, 1024] x [4096, 1024]^T, the up-projection of a transformer block's feed forward: rows sampled against
    the oracle; the bias epilogue agrees with the same bias folded into the product as one more column of K."""
    M, N, K = 16384, 4096, 1024
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(M, K, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=gen) / 32).bfloat16()
    b = (0.1 * torch.randn(N, device="cuda", generator=gen)).bfloat16()
    y, _ = abi.linear_bias_act_fwd(x, w, b, abi.ACT_GELU)
    idx = torch.linspace(0, M - 1, 40).long().cuda()
    ref = O.linear_act(x[idx].float().cpu().numpy(), w.float().cpu().numpy(), b.float().cpu().numpy(), O.ACT_GELU)
    gemm_check(y[idx], ref["y"], x[idx].float().cpu().numpy(), w.float().cpu().numpy(), b.float().cpu().numpy(), "sampled rows")
    assert torch.equal(y, abi.linear_bias_act_fwd(x, w, b, abi.ACT_GELU)[0])           # deterministic
    # the bias as one more column of K (x' = [x | 1 0...], w' = [w | b 0...]) is the same sum: bias path == plain GEMM path
    xp = torch.cat([x, torch.zeros(M, 8, device="cuda", dtype=torch.bfloat16)], 1); xp[:, K] = 1
    wp = torch.cat([w, torch.zeros(N, 8, device="cuda", dtype=torch.bfloat16)], 1); wp[:, K] = b
    z_bias, _ = abi.linear_bias_act_fwd(x, w, b, abi.ACT_NONE)
    z_col, _ = abi.linear_bias_act_fwd(xp.contiguous(), wp.contiguous(), None, abi.ACT_NONE)
    gemm_check(z_col[idx], z_bias[idx].float().cpu().numpy().astype(np.float64), x[idx].float().cpu().numpy(), w.float().cpu().numpy(),
               b.float().cpu().numpy(), "bias as a column of K")


def test_argument_checks():
    L = abi.lib()
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 4, 8, 8, abi.F32, 0, None, 0, None) == -3      # fp32 is not taken
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 4, 12, 8, abi.BF16, 0, None, 0, None) == -2    # N % 8
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 0, 8, 8, abi.BF16, 0, None, 0, None) == 0      # empty
    assert L.nb2_linear_bias_act_fwd(None, None, None, None, None, 4, 8, 8, abi.BF16, 0, None, 0, None) == -1     # NULL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("act_type,act", [(7, "gelu"), (6, "silu"), (0, "none")])      # Nott::Activation::Type: GeLU = 7, SiLU = 6
def test_linear_module_forward_and_backward_match_torch(dtype, act_type, act):
    """The C++ drop-in for the FC layer (parameter names of torch::nn::Linear, activation fused) against
    torch.nn.functional.linear + activation + autograd on the same GPU tensors."""
    import torch.nn.functional as F
    from thot_b200 import _nott_b200_host as host
    B, S, K, N = 3, 50, 256, 512
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(B, S, K, generator=gen).to(dtype).cuda(); w = (torch.randn(N, K, generator=gen) / 16).to(dtype).cuda()
    b = (0.1 * torch.randn(N, generator=gen)).to(dtype).cuda(); dy = torch.randn(B, S, N, generator=gen).to(dtype).cuda()
    names, out = host.linear_module_step(x, w, b, act_type, dy)
    assert names == ["weight", "bias"]
    xr, wr, br = (t.float().clone().requires_grad_(True) for t in (x, w, b))
    z = F.linear(xr, wr, br)
    yr = {"gelu": F.gelu, "silu": F.silu, "none": lambda t: t}[act](z)
    yr.backward(dy.float())
    rtol, atol = (2e-2, 2e-2) if dtype == torch.bfloat16 else (1e-4, 1e-4)
    for got, want in zip(out, (yr, xr.grad, wr.grad, br.grad)):
        torch.testing.assert_close(got.float(), want.detach(), rtol=rtol, atol=atol * max(1.0, float(want.abs().max())))
    if dtype == torch.bfloat16:      # the forward is the fused tensor-core call: 2 bf16 ulp of the fp64 oracle
        ref = O.linear_act(x.float().cpu().numpy().reshape(-1, K), w.float().cpu().numpy(), b.float().cpu().numpy(),
                           {"gelu": O.ACT_GELU, "silu": O.ACT_SILU, "none": O.ACT_NONE}[act])
        check(out[0].reshape(-1, N), ref["y"], "module y")
