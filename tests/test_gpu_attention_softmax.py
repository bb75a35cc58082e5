"""Attention probabilities (scale, key padding, additive mask, causal, softmax) in one kernel:
C ABI against the reference's ScaledDotProductKernel goldens and the CPU oracle, and the C++
drop-in module against the same arithmetic written with torch ops."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from tests.gpu_util import check, make, to_dev
from tests.test_oracle_golden import ATTN_CASES
from thot_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(ATTN_CASES))
def test_golden_reference_kernel(golden_dir, name):
    z = np.load(golden_dir / "attention_softmax.npz")
    pk, mk, causal = ATTN_CASES[name]
    scores = to_dev(z["scores"], torch.float32)
    S = scores.shape[-1]
    padding = torch.from_numpy(z[pk]).cuda() if pk else None
    mask = torch.from_numpy(z[mk]).cuda() if mk else None
    attn = abi.attention_softmax_fwd(scores, 1.0 / math.sqrt(S), padding, mask, causal)
    check(attn, z[f"{name}_attn_f64"], "attn")
    ds = abi.attention_softmax_bwd(attn, to_dev(z["dattn"], torch.float32), 1.0 / math.sqrt(S))
    check(ds, z[f"{name}_dscores_f64"], "dscores")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,T,S,mask_rank,use_padding,causal", [
    (2, 4, 128, 128, 0, False, True),        # one warp per row
    (1, 2, 64, 512, 2, True, False),
    (2, 2, 16, 2048, 3, False, False),       # several warps per row
    (1, 1, 8, 8192, 4, True, False),         # the widest register-row shape for fp32
    (2, 3, 9, 77, 4, True, True),            # ragged length: the three-sweep kernel
    (1, 1, 3, 16400, 0, False, False),       # beyond the register-row shapes
])
def test_against_oracle(dtype, B, H, T, S, mask_rank, use_padding, causal):
    scores, sn = make((B, H, T, S), 1, dtype, 2.0)
    dattn, dn = make((B, H, T, S), 2, dtype)
    mask_shape = {0: None, 2: (T, S), 3: (B, T, S), 4: (B, H, T, S)}[mask_rank]
    mask, mn = make(mask_shape, 3, dtype) if mask_shape else (None, None)
    padding = None
    if use_padding:
        padding = torch.zeros(B, S, dtype=torch.bool)
        padding[-1, S - S // 3:] = True
    scale = 1.0 / math.sqrt(64)
    attn = abi.attention_softmax_fwd(scores, scale, None if padding is None else padding.cuda(), mask, causal)
    ref = O.attention_softmax(sn, scale, None if padding is None else padding.numpy(), mn, causal, None)
    check(attn.reshape(-1, S), ref["attn"].reshape(-1, S), "attn")
    assert torch.allclose(attn.float().sum(-1), torch.ones(B, H, T, device="cuda"), atol=2e-2 if dtype == torch.bfloat16 else 1e-5)
    # backward from the probabilities the kernel itself stored (bf16: rounded), as autograd would run it
    an = attn.float().cpu().numpy().astype(np.float64)
    dot = (an * dn).sum(-1, keepdims=True)
    ds = abi.attention_softmax_bwd(attn, dattn, scale)
    check(ds.reshape(-1, S), (scale * an * (dn - dot)).reshape(-1, S), "dscores")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,T,S,mask_rank,use_padding,causal,with_noise", [
    (2, 4, 33, 128, 3, False, False, False),      # one warp per row; 66 (batch, position) pairs do not fill the groups evenly
    (1, 16, 40, 1024, 2, True, True, False),      # a [T, S] mask under padding and the causal cut
    (3, 5, 7, 2048, 3, True, False, True),        # several warps per row, odd head count, dropout noise
    (2, 8, 300, 256, 3, False, True, True),       # more pairs than one pass of the grid covers
])
def test_mask_shared_by_the_heads_kept_per_position(dtype, B, H, T, S, mask_rank, use_padding, causal, with_noise):
    """With one mask row serving all heads of a (batch, position) pair the forward walks the heads innermost and keeps
    the row in registers.  Checked against the oracle, and bit for bit against the same call with the mask expanded to
    [B, H, T, S] (a head stride, so rows go in memory order and the mask is read per row)."""
    scores, sn = make((B, H, T, S), 11, dtype, 2.0)
    mask, mn = make((T, S) if mask_rank == 2 else (B, T, S), 12, dtype)
    padding = None
    if use_padding:
        padding = torch.zeros(B, S, dtype=torch.bool)
        padding[-1, S - S // 3:] = True
    pad_dev = None if padding is None else padding.cuda()
    noise = None
    if with_noise:
        noise = ((torch.rand(B, H, T, S, generator=torch.Generator().manual_seed(13)) >= 0.25).float() * 1.25).to(dtype).cuda()
    scale = 1.0 / math.sqrt(64)
    full = (mask if mask_rank == 3 else mask[None]).reshape(-1, 1, T, S).expand(B, H, T, S).contiguous()
    before = abi.attention_softmax_order(2)            # these shapes are too small for the size rule to pick it
    try:
        got = abi.attention_softmax_fwd(scores, scale, pad_dev, mask, causal, noise=noise)
    finally:
        abi.attention_softmax_order(before)
    flat = abi.attention_softmax_fwd(scores, scale, pad_dev, full, causal, noise=noise)
    if with_noise:
        assert torch.equal(got[0], flat[0]) and torch.equal(got[1], flat[1])
        attn = got[1]
    else:
        assert torch.equal(got, flat)
        attn = got
    ref = O.attention_softmax(sn, scale, None if padding is None else padding.numpy(), mn, causal, None)
    check(attn.reshape(-1, S), ref["attn"].reshape(-1, S), "attn")


def test_a_fully_masked_row_is_nan_like_the_reference():
    scores, _ = make((1, 1, 2, 64), 1, torch.float32)
    padding = torch.ones(1, 64, dtype=torch.bool, device="cuda")
    attn = abi.attention_softmax_fwd(scores, 0.125, padding)
    assert torch.isnan(attn).all()
    assert abi.lib().nb2_attention_softmax_fwd(None, None, None, 0, 0, None, 1, 1, 1, 8, 1.0, 0, 0, None) == -1   # NULL
    assert abi.lib().nb2_attention_softmax_fwd(None, None, None, 0, 0, None, 1, 1, 0, 8, 1.0, 0, 0, None) == 0    # empty
    assert abi.lib().nb2_attention_softmax_fwd(None, None, None, 0, 0, None, 1, 1, 1, 8, 1.0, 0, 7, None) == -3   # dtype


@pytest.mark.parametrize("causal", [False, True])
def test_scaled_dot_product_module_matches_torch_ops(causal):
    """The C++ drop-in for the reference's ScaledDotProductKernel against the reference's own sequence
    of torch ops (kernel.hpp:26-95) run on the same GPU in fp32, values and gradients."""
    from thot_b200 import _nott_b200_host as host
    B, H, T, S, hd = 2, 3, 40, 56, 32
    q, _ = make((B, H, T, hd), 1, torch.float32); k, _ = make((B, H, S, hd), 2, torch.float32); v, _ = make((B, H, S, hd), 3, torch.float32)
    mask, _ = make((B, T, S), 4, torch.float32)
    padding = torch.zeros(B, S, dtype=torch.bool, device="cuda"); padding[0, -9:] = True
    dout, _ = make((B, H, T, hd), 5, torch.float32)

    def reference(q, k, v):
        scores = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(hd)
        scores = scores.masked_fill(padding[:, None, None, :], float("-inf")) + mask[:, None]
        if causal:
            scores = scores.masked_fill(torch.ones(T, S, dtype=torch.bool, device="cuda").triu(1), float("-inf"))
        return torch.matmul(torch.softmax(scores, -1), v)

    grads = []
    outs = []
    for fn in (reference, lambda q, k, v: host.scaled_dot_product(q, k, v, mask, padding, causal)):
        qi, ki, vi = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = fn(qi, ki, vi)
        out.backward(dout)
        outs.append(out.detach()); grads.append((qi.grad, ki.grad, vi.grad))
    torch.testing.assert_close(outs[1], outs[0], rtol=1e-5, atol=1e-5)
    for got, want in zip(grads[1], grads[0]):
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):                     # std::invalid_argument, as the reference throws
        host.attention_softmax(torch.zeros(B, H, T, S, device="cuda"), torch.zeros(T + 1, S, device="cuda"), None, 1.0, False)


def test_full_size_properties_bf16():
    """[16, 16, 1024, 1024] bf16, causal (the measured case): every row sums to 1, nothing attends to a
    later column, reruns are bit-identical, and sampled rows match the oracle."""
    B, H, T, S = 16, 16, 1024, 1024
    gen = torch.Generator(device="cuda").manual_seed(11)
    scores = torch.randn(B, H, T, S, device="cuda", generator=gen).to(torch.bfloat16)
    attn = abi.attention_softmax_fwd(scores, 0.125, causal=True)
    sums = attn.float().sum(-1)
    assert torch.allclose(sums, torch.ones_like(sums), atol=2e-2)
    assert not torch.triu(attn[3, 5], 1).any() and not torch.triu(attn[-1, -1], 1).any()
    assert torch.equal(attn, abi.attention_softmax_fwd(scores, 0.125, causal=True))
    for (b, h) in ((0, 0), (7, 9), (15, 15)):
        # sampled rows t = 0, 97, ...: the definition, with the causal cut, in fp64 on the host
        rows = np.arange(0, T, 97)
        x = scores[b, h, ::97].float().cpu().numpy().astype(np.float64) * 0.125
        x[np.arange(S)[None, :] > rows[:, None]] = -np.inf
        e = np.exp(x - x.max(-1, keepdims=True)); ref = e / e.sum(-1, keepdims=True)
        check(attn[b, h, ::97], ref, f"rows of ({b},{h})")
    d = torch.randn(B, H, T, S, device="cuda", generator=gen).to(torch.bfloat16)
    ds = abi.attention_softmax_bwd(attn, d, 0.125)
    # softmax backward is orthogonal to the all-ones direction: every row of dscores sums to ~0
    assert ds.float().sum(-1).abs().max() < 2e-2
    assert not torch.triu(ds[2, 2], 1).any()


# ---- the dropout that follows the softmax, in the same pass (kernel.hpp:94; dropout.hpp:32-51)
@pytest.mark.parametrize("name", ["plain", "mask3_padding_causal"])
def test_dropout_golden_reference_modules(golden_dir, name):
    """Golden = the reference's ScaledDotProductKernel probabilities followed by its HardDropout module
    (input * N(1, sqrt(p/(1-p)))), with the noise tensor that module drew."""
    z = np.load(golden_dir / "attention_softmax_dropout.npz")
    scores = to_dev(z["scores"], torch.float32)
    S = scores.shape[-1]
    use = name != "plain"
    padding = torch.from_numpy(z["padding"]).cuda() if use else None
    mask = torch.from_numpy(z["mask3"]).cuda() if use else None
    noise = to_dev(z[f"{name}_noise_f32"], torch.float32)
    out, pre = abi.attention_softmax_fwd(scores, 1.0 / math.sqrt(S), padding, mask, use, noise=noise)
    check(pre, z[f"{name}_attn_f64"], "attn")
    check(out, z[f"{name}_out_f32"], "dropped (reference fp32)")
    check(out, z[f"{name}_attn_f64"].astype(np.float64) * z[f"{name}_noise_f32"], "dropped")
    ds = abi.attention_softmax_bwd(pre, to_dev(z["dout"], torch.float32), 1.0 / math.sqrt(S), noise=noise)
    check(ds, z[f"{name}_dscores_f32"], "dscores (reference fp32)")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,T,S,use_mask,causal,bernoulli", [
    (2, 4, 128, 128, False, True, True),
    (1, 2, 64, 512, True, False, False),
    (2, 2, 16, 2048, True, False, True),
    (2, 3, 9, 77, True, True, False),         # ragged length: the three-sweep kernel
])
def test_dropout_against_oracle(dtype, B, H, T, S, use_mask, causal, bernoulli):
    p = 0.2
    scores, sn = make((B, H, T, S), 1, dtype, 2.0)
    dout, dn = make((B, H, T, S), 2, dtype)
    mask, mn = make((B, T, S), 3, dtype) if use_mask else (None, None)
    gen = torch.Generator().manual_seed(9)
    if bernoulli:      # torch::nn::Dropout's form: keep mask over 1-p (1.25 is a bf16 number)
        noise_t = (torch.rand(B, H, T, S, generator=gen) >= p).float() / (1 - p)
    else:              # the multiplicative-noise module: N(1, sqrt(p/(1-p)))
        noise_t = 1 + math.sqrt(p / (1 - p)) * torch.randn(B, H, T, S, generator=gen)
    noise_t = noise_t.to(dtype)
    nn_ = noise_t.float().numpy()
    scale = 0.125
    out, pre = abi.attention_softmax_fwd(scores, scale, None, mask, causal, noise=noise_t.cuda())
    ref = O.attention_softmax(sn, scale, None, mn, causal, None)
    check(pre.reshape(-1, S), ref["attn"].reshape(-1, S), "attn before the noise")
    # the dropped probabilities are the STORED probabilities times the noise, rounded once
    pn = pre.float().cpu().numpy().astype(np.float64)
    check(out.reshape(-1, S), (pn * nn_).reshape(-1, S), "dropped")
    assert torch.equal(pre, abi.attention_softmax_fwd(scores, scale, None, mask, causal))         # same bits as the plain call
    out_only, none = abi.attention_softmax_fwd(scores, scale, None, mask, causal, noise=noise_t.cuda(), want_pre=False)
    assert none is None and torch.equal(out_only, out)
    # backward: the gradient of the probabilities is dout * noise as a tensor of the activation type
    ds = abi.attention_softmax_bwd(pre, dout, scale, noise=noise_t.cuda())
    if dtype == torch.float32:
        dattn = (dn.astype(np.float32) * nn_).astype(np.float64)
    else:
        from tests import tol
        dattn = tol.bf16_bits_to_f32(tol.to_bf16_bits(dn.astype(np.float64) * nn_)).astype(np.float64).reshape(dn.shape)
    dot = (pn * dattn).sum(-1, keepdims=True)
    check(ds.reshape(-1, S), (scale * pn * (dattn - dot)).reshape(-1, S), "dscores")
    # and it equals the two-step form: a separate multiply, then the plain softmax backward
    two_step = abi.attention_softmax_bwd(pre, (dout.float() * noise_t.cuda().float()).to(dtype), scale)
    assert torch.equal(ds, two_step)


def test_dropout_module_matches_torch_ops_given_the_same_noise():
    from thot_b200 import _nott_b200_host as host
    B, H, T, S, hd = 2, 3, 40, 56, 32
    q, _ = make((B, H, T, hd), 1, torch.float32); k, _ = make((B, H, S, hd), 2, torch.float32); v, _ = make((B, H, S, hd), 3, torch.float32)
    dout, _ = make((B, H, T, hd), 5, torch.float32)
    p = 0.3
    gen = torch.Generator(device="cuda").manual_seed(3)
    noise = (torch.rand(B, H, T, S, device="cuda", generator=gen) >= p).float() / (1 - p)

    def reference(q, k, v):
        attn = torch.softmax(torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(hd), -1)
        return torch.matmul(attn * noise, v)

    res = []
    for fn in (reference, lambda q, k, v: host.scaled_dot_product_dropout(q, k, v, noise, p, False)):
        qi, ki, vi = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = fn(qi, ki, vi)
        out.backward(dout)
        res.append((out.detach(), qi.grad, ki.grad, vi.grad))
    for got, want in zip(res[1], res[0]):
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    # the module's own draw: about a fraction p of the probabilities is dropped and the rest is scaled by 1/(1-p)
    vi = torch.eye(S, device="cuda").expand(B, H, S, S).contiguous()
    kept = host.scaled_dot_product_dropout(q, k, vi, None, p, False)       # value = identity: the output is attn * noise
    plain = torch.softmax(torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(hd), -1)
    ratio = kept / plain
    dropped = (kept == 0).float().mean().item()
    assert abs(dropped - p) < 0.03
    assert torch.allclose(ratio[kept != 0], torch.full_like(ratio[kept != 0], 1 / (1 - p)), rtol=1e-4)


def test_row_order_setting_round_trip_and_size_rule():
    """The order knob returns the previous value and rejects anything but 0..2; with the default setting a large shared
    mask case and a small one both match the memory-order result bit for bit (whichever order the size rule picks)."""
    assert abi.attention_softmax_order(1) == 0
    assert abi.attention_softmax_order(0) == 1
    with pytest.raises(abi.Nb2Error):
        abi.attention_softmax_order(3)
    assert abi.attention_softmax_order(0) == 0
    for (B, H, T, S) in ((16, 4, 512, 128), (1, 8, 4, 128)):          # 8192 pairs: heads innermost; 4 pairs: memory order
        scores, _ = make((B, H, T, S), 21, torch.bfloat16, 2.0)
        mask, _ = make((B, T, S), 22, torch.bfloat16)
        auto = abi.attention_softmax_fwd(scores, 0.125, None, mask, False)
        abi.attention_softmax_order(1)
        try:
            flat = abi.attention_softmax_fwd(scores, 0.125, None, mask, False)
        finally:
            abi.attention_softmax_order(0)
        assert torch.equal(auto, flat)
