"""The C++ libtorch host layer (thot_b200/host/nott_b200.hpp: autograd functions and drop-in
modules) through its Python binding, against libtorch's own CUDA ops run in fp32 (the ops the
reference executes on a GPU) and the CPU oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import check, make

pytestmark = pytest.mark.gpu

ACT = {"Identity": 0, "SiLU": 6, "GeLU": 7, "SwiGLU": 9, "Swish": 13, "ReLU": 1}     # Nott::Activation::Type order
NB2 = {0: 0, 7: 1, 6: 2, 13: 2}


@pytest.fixture(scope="module")
def host():
    import torch  # noqa: F401  (libtorch must be loaded first)
    from thot_b200 import _nott_b200_host as h
    return h


def torch_act(z, code):
    return {0: z, 1: F.gelu(z), 2: F.silu(z)}[code]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", [0, 1, 2])
def test_layernorm_function_autograd(host, dtype, act):
    x, xn = make((4, 37, 1024), 1, dtype)
    dy, dyn = make((4, 37, 1024), 2, dtype)
    w, wn = make((1024,), 3, dtype, 0.02, 1.0)
    b, bn = make((1024,), 4, dtype, 0.02)
    x.requires_grad_(True); w.requires_grad_(True); b.requires_grad_(True)
    y = host.layernorm_act(x, w, b, 1e-5, act)
    assert y.shape == x.shape and y.dtype == dtype
    y.backward(dy)
    ref = O.layernorm_act(xn.reshape(-1, 1024), wn, bn, dyn.reshape(-1, 1024), 1e-5, act)
    check(y.detach().reshape(-1, 1024), ref["y"], "y")
    check(x.grad.reshape(-1, 1024), ref["dx"], "dx")
    assert w.grad.dtype == dtype and b.grad.dtype == dtype
    if dtype == torch.float32:
        tol.long_sum_close(w.grad.cpu().numpy(), ref["dgamma"], 148)
        tol.long_sum_close(b.grad.cpu().numpy(), ref["dbeta"], 148)
        # libtorch's own CUDA kernels in fp32: the ops the reference runs on a GPU
        x2 = x.detach().clone().requires_grad_(True)
        y2 = torch_act(F.layer_norm(x2, (1024,), w.detach(), b.detach(), 1e-5), act)
        y2.backward(dy)
        tol.fp32_close_adjudicated(y.detach().cpu().numpy().reshape(-1, 1024), y2.detach().cpu().numpy().reshape(-1, 1024), ref["y"])
        tol.fp32_close_adjudicated(x.grad.cpu().numpy().reshape(-1, 1024), x2.grad.cpu().numpy().reshape(-1, 1024), ref["dx"])
    else:
        tol.bf16_ulp_close(tol.to_bf16_bits(w.grad.float().cpu().numpy()), ref["dgamma"])


def test_modules_keep_reference_parameter_names_and_errors(host):
    x, xn = make((6, 512), 5, torch.float32)
    dy, dyn = make((6, 512), 6, torch.float32)
    names, out = host.layernorm_module_step(512, 1e-5, True, ACT["GeLU"], x, dy)
    assert names == ["weight", "bias"]                       # checkpoint keys of torch::nn::LayerNorm
    ref = O.layernorm_act(xn, np.ones(512, np.float32), np.zeros(512, np.float32), dyn, 1e-5, O.ACT_GELU)
    check(out[0], ref["y"], "module y")
    check(out[1], ref["dx"], "module dx")
    tol.long_sum_close(out[2].cpu().numpy(), ref["dgamma"], 6)
    tol.long_sum_close(out[3].cpu().numpy(), ref["dbeta"], 6)
    names, out = host.layernorm_module_step(512, 1e-12, False, ACT["Identity"], x, dy)
    assert names == []
    check(out[0], O.layernorm_act(xn, None, None, None, 1e-12)["y"], "no-affine y")
    names, out = host.rmsnorm_module_step(512, 1e-6, True, ACT["SiLU"], x, dy)
    assert names == ["weight"]                                # Mamba RMSNorm registers "weight"
    ref = O.rmsnorm_act(xn, np.ones(512, np.float32), dyn, 1e-6, O.ACT_SILU)
    check(out[0], ref["y"], "rms y")
    check(out[1], ref["dx"], "rms dx")
    msgs = host.module_errors()
    assert len(msgs) == 3 and "positive embedding dimension" in msgs[0] and "defined input" in msgs[1] and "CUDA" in msgs[2]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_apply_dispatch(host, dtype):
    x, xn = make((5, 96), 7, dtype, 2.0)
    dy, dyn = make((5, 96), 8, dtype)
    for name, code in (("GeLU", O.ACT_GELU), ("SiLU", O.ACT_SILU), ("Swish", O.ACT_SILU)):
        xi = x.clone().requires_grad_(True)
        y = host.apply(ACT[name], xi)
        y.backward(dy)
        ref = O.act(xn, dyn, code)
        check(y.detach(), ref["y"], name)
        check(xi.grad, ref["dx"], name + " grad")
    xi = x.clone().requires_grad_(True)
    y = host.apply(ACT["SwiGLU"], xi)                         # [5, 96] -> [5, 48]
    assert y.shape == (5, 48)
    y.backward(dy[:, :48].contiguous())
    ref = O.silu_gate(xn[:, :48], xn[:, 48:], dyn[:, :48])
    check(y.detach(), ref["out"], "swiglu")
    check(xi.grad[:, :48].contiguous(), ref["da"], "swiglu da")
    check(xi.grad[:, 48:].contiguous(), ref["db"], "swiglu db")
    assert host.apply(ACT["Identity"], x) is not None
    with pytest.raises(ValueError):                           # std::invalid_argument
        host.apply(ACT["ReLU"], x)


def test_mamba_gate_embedding_and_rotary(host):
    gate, gn = make((3, 7, 64), 9, torch.bfloat16)
    up, un = make((3, 7, 64), 10, torch.bfloat16)
    out = host.silu_gate(gate, up)
    check(out.reshape(-1, 64), O.silu_gate(gn.reshape(-1, 64), un.reshape(-1, 64), None)["out"], "mamba gate")

    table, _ = make((50, 24), 11, torch.float32, 0.02)
    table.requires_grad_(True)
    ids = torch.randint(0, 50, (4, 9), device="cuda")
    emb = host.embedding(table, ids)
    assert torch.equal(emb, table.detach()[ids])             # bit-exact gather
    dout, dn = make((4, 9, 24), 12, torch.float32)
    emb.backward(dout)
    check(table.grad, O.embedding_bwd(dn.reshape(-1, 24), ids.cpu().numpy(), 50), "dtable")

    q, qn = make((2, 16, 4, 128), 13, torch.bfloat16)
    q.requires_grad_(True)
    cs = host.rotary_table(16, 128, 10000.0, torch.device("cuda"))
    rq = host.rotary(q, cs)
    check(rq.detach(), O.rope_apply(qn, cs.cpu().numpy()), "rotary")
    dq, dqn = make((2, 16, 4, 128), 14, torch.bfloat16)
    rq.backward(dq)
    check(q.grad, O.rope_apply(dqn, cs.cpu().numpy(), inverse=True), "rotary grad")


def test_autocast_runs_layernorm_in_fp32(host):
    x, xn = make((8, 256), 15, torch.bfloat16)
    dy, _ = make((8, 256), 16, torch.float32)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        names, out = host.layernorm_module_step(256, 1e-5, True, ACT["Identity"], x.float(), dy)
    assert out[0].dtype == torch.float32


@pytest.mark.parametrize("rms", [False, True])
def test_residual_add_norm_autograd(host, rms):
    dtype = torch.float32
    a, an = make((3, 50, 1024), 21, dtype); b, bn = make((3, 50, 1024), 22, dtype)
    w, wn = make((1024,), 23, dtype, 0.02, 1.0); bias, biasn = make((1024,), 24, dtype, 0.02)
    dy, dyn = make((3, 50, 1024), 25, dtype); ds, dsn = make((3, 50, 1024), 26, dtype)
    a.requires_grad_(True); b.requires_grad_(True); w.requires_grad_(True); bias.requires_grad_(True)
    s, y = host.add_norm(a, b, w, None if rms else bias, 1e-6 if rms else 1e-5, rms)
    ((y * dy).sum() + (s * ds).sum()).backward()
    ref = O.add_norm("rms" if rms else "ln", an.reshape(-1, 1024), bn.reshape(-1, 1024), wn, None if rms else biasn,
                     dyn.reshape(-1, 1024), dsn.reshape(-1, 1024), 1e-6 if rms else 1e-5)
    assert torch.equal(s.detach(), a.detach() + b.detach())
    check(y.detach().reshape(-1, 1024), ref["y"], "y")
    check(a.grad.reshape(-1, 1024), ref["dx"], "da")
    assert torch.equal(a.grad, b.grad)
    tol.long_sum_close(w.grad.cpu().numpy(), ref["dgamma"], 150)
    if not rms:
        tol.long_sum_close(bias.grad.cpu().numpy(), ref["dbeta"], 150)
    # only the normalised output is used downstream: the residual gradient is absent
    a2 = a.detach().clone().requires_grad_(True)
    s2, y2 = host.add_norm(a2, b.detach(), w.detach(), None if rms else bias.detach(), 1e-6 if rms else 1e-5, rms)
    y2.backward(dy)
    ref2 = O.add_norm("rms" if rms else "ln", an.reshape(-1, 1024), bn.reshape(-1, 1024), wn, None if rms else biasn,
                      dyn.reshape(-1, 1024), None, 1e-6 if rms else 1e-5)
    check(a2.grad.reshape(-1, 1024), ref2["dx"], "da without residual gradient")
