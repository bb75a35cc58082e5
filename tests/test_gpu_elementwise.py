"""Stand-alone GELU/SiLU and the SiLU gate (SwiGLU / Mamba forms) through the C ABI."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from tests.gpu_util import check, make, to_dev
from thot_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,code", [("gelu", abi.ACT_GELU), ("silu", abi.ACT_SILU)])
def test_activation_golden(golden_dir, name, code):
    g = np.load(golden_dir / "act_gelu_silu.npz")
    x, dy = to_dev(g["x"], torch.float32), to_dev(g["dy"], torch.float32)
    check(abi.act_fwd(x, code), g[f"{name}_y_f32"], name + " y")
    check(abi.act_bwd(x, dy, code), g[f"{name}_dx_f32"], name + " dx")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("code", [abi.ACT_GELU, abi.ACT_SILU])
@pytest.mark.parametrize("n", [1, 7, 1000, 4099, 1 << 20, (1 << 22) + 3])
def test_activation_sizes_and_tails(dtype, code, n):
    x, xn = make((n,), n, dtype, 2.0)
    dy, dyn = make((n,), n + 1, dtype)
    ref = O.act(xn, dyn, code)
    check(abi.act_fwd(x, code), ref["y"], "y")
    check(abi.act_bwd(x, dy, code), ref["dx"], "dx")


def test_activation_unaligned_pointer():
    base, bn = make((5001,), 3, torch.bfloat16, 2.0)
    x = base[1:]
    assert x.data_ptr() % 16 != 0
    check(abi.act_fwd(x, abi.ACT_GELU), O.act(bn[1:], None, O.ACT_GELU)["y"], "unaligned gelu")


def test_silu_gate_golden_swiglu_and_mamba(golden_dir):
    g = np.load(golden_dir / "silu_gate.npz")
    inp, dy = to_dev(g["input"], torch.float32), to_dev(g["dy"], torch.float32)
    H = inp.shape[1] // 2
    a, b = inp[:, :H], inp[:, H:]                       # SwiGLU: strided halves of one tensor
    check(abi.silu_gate_fwd(a, b), g["swiglu_out_f32"], "swiglu out")
    dinp = torch.empty_like(inp)
    abi.silu_gate_bwd(a, b, dy, dinp[:, :H], dinp[:, H:])
    check(dinp, g["swiglu_dinput_f32"], "swiglu dinput")
    ac, bc = a.contiguous(), b.contiguous()             # Mamba: separate tensors
    check(abi.silu_gate_fwd(ac, bc), g["mamba_out_f32"], "mamba out")
    da, db = abi.silu_gate_bwd(ac, bc, dy)
    check(da, g["mamba_dgate_f32"], "mamba dgate")
    check(db, g["mamba_dup_f32"], "mamba dup")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(1, 1), (3, 7), (5, 40), (130, 1376), (257, 11008), (6, 11009)])
def test_silu_gate_shapes(dtype, rows, H):
    inp, inn = make((rows, 2 * H), rows * 31 + H, dtype, 1.5)
    dy, dyn = make((rows, H), rows * 37 + H, dtype)
    a, b = inp[:, :H], inp[:, H:]
    ref = O.silu_gate(inn[:, :H], inn[:, H:], dyn)
    check(abi.silu_gate_fwd(a, b), ref["out"], "out")
    da, db = abi.silu_gate_bwd(a, b, dy)
    check(da, ref["da"], "da")
    check(db, ref["db"], "db")


def test_config3_silu_gate_bf16_full_size_sampled():
    """a,b[65536,11008] bf16: full-size run, a scattered row sample against the oracle."""
    rows, H = 65536, 11008
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(rows, H, device="cuda", generator=gen).bfloat16()
    b = torch.randn(rows, H, device="cuda", generator=gen).bfloat16()
    dy = torch.randn(rows, H, device="cuda", generator=gen).bfloat16()
    out = abi.silu_gate_fwd(a, b)
    da, db = abi.silu_gate_bwd(a, b, dy)
    idx = torch.linspace(0, rows - 1, 40).long().cuda()
    ref = O.silu_gate(a[idx].float().cpu().numpy(), b[idx].float().cpu().numpy(), dy[idx].float().cpu().numpy())
    check(out[idx], ref["out"], "out")
    check(da[idx], ref["da"], "da")
    check(db[idx], ref["db"], "db")
    # idempotence of the launch: same inputs, same bits
    assert torch.equal(out, abi.silu_gate_fwd(a, b))
