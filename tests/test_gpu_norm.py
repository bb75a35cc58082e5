"""LayerNorm / RMSNorm (+GELU/SiLU) CUDA kernels, called through the C ABI, against the
CPU oracle, the committed reference outputs and (when built) the reference itself."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from oracle import reference as R
from tests import tol
from tests.gpu_util import bits, check, make, to_dev
from thot_b200 import abi

pytestmark = pytest.mark.gpu

NORM_CASES = ["ln_d512_none", "ln_d1024_gelu", "ln_d7_silu_eps1e-12", "ln_d2048_gelu_noaffine",
              "ln_d768_gelu_bf16", "rms_d4096_none_bf16", "rms_d768_silu", "rms_d33_gelu_noweight"]


def run_gpu(kind, x, gamma, beta, dy, eps, act):
    if kind == "ln":
        y, mean, rstd = abi.layernorm_fwd(x, gamma, beta, eps, act)
        dx, gb = abi.layernorm_bwd(x, dy, gamma, beta, mean, rstd, act, want_param_grads=gamma is not None)
        out = dict(y=y, dx=dx, mean=mean, rstd=rstd)
        if gb is not None:
            out["dgamma"], out["dbeta"] = gb[0], gb[1]
        return out
    y, rstd = abi.rmsnorm_fwd(x, gamma, eps, act)
    dx, dw = abi.rmsnorm_bwd(x, dy, gamma, rstd, act, want_param_grads=gamma is not None)
    out = dict(y=y, dx=dx, rstd=rstd)
    if dw is not None:
        out["dweight"] = dw
    return out


@pytest.mark.parametrize("name", NORM_CASES)
def test_golden_reference_outputs(golden_dir, name):
    z = np.load(golden_dir / f"{name}.npz")
    g = {k: z[k] for k in z.files}
    dtype = torch.bfloat16 if bool(g["bf16"]) else torch.float32
    kind = str(g["kind"])
    x, dy = to_dev(g["x"], dtype), to_dev(g["dy"], dtype)
    gamma = to_dev(g["gamma"], dtype) if "gamma" in g else None
    beta = to_dev(g["beta"], dtype) if "beta" in g else None
    out = run_gpu(kind, x, gamma, beta, dy, float(g["eps"]), int(g["act"]))
    check(out["y"], g["y_f32"], "y")
    check(out["dx"], g["dx_f32"], "dx")
    for k in ("dgamma", "dbeta", "dweight"):
        if k in out:
            # the parameter gradients leave the library as fp32 sums whatever the activation dtype
            tol.long_sum_close(out[k].cpu().numpy(), g[f"{k}_f64x"], int(g["rows"]), ref32=g[f"{k}_f32"])


SHAPES = [(1, 1), (3, 7), (33, 512), (5, 513), (300, 768), (64, 1024), (37, 2048), (19, 4096),
          (3, 8191), (9, 8192), (2, 16384), (4, 20000),
          (41, 384), (310, 1536), (150, 3072), (70, 6144),       # 3 * 2^k: three vectors per thread in the ring kernels
          (77, 640), (330, 1280), (160, 2560), (75, 5120), (40, 10240),    # 5 * 2^k: five vectors, or 160/320-thread row groups
          (230, 1792), (120, 3584), (60, 7168), (11, 14336)]               # 7 * 2^k: 224/448-thread row groups


@pytest.mark.parametrize("kind", ["ln", "rms"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", [abi.ACT_NONE, abi.ACT_GELU, abi.ACT_SILU])
def test_against_oracle_over_shapes(kind, dtype, act):
    eps = 1e-5 if kind == "ln" else 1e-6
    for i, (rows, D) in enumerate(SHAPES):
        seed = 100 + i
        x, xn = make((rows, D), seed, dtype)
        dy, dyn = make((rows, D), seed + 1000, dtype)
        gamma, gn = make((D,), seed + 2000, dtype, 0.02, 1.0)
        beta, bn = make((D,), seed + 3000, dtype, 0.02) if kind == "ln" else (None, None)
        out = run_gpu(kind, x, gamma, beta, dy, eps, act)
        ref = O.layernorm_act(xn, gn, bn, dyn, eps, act) if kind == "ln" else O.rmsnorm_act(xn, gn, dyn, eps, act)
        what = f"{kind} {dtype} act={act} rows={rows} D={D}"
        check(out["y"], ref["y"], what + " y")
        check(out["dx"], ref["dx"], what + " dx")
        tol.fp32_close(out["rstd"].cpu().numpy(), ref["rstd"], rtol=2e-6, atol=0)
        if kind == "ln":
            tol.fp32_close(out["mean"].cpu().numpy(), ref["mean"], rtol=1e-5, atol=1e-6)
        for k in ("dgamma", "dbeta", "dweight"):
            if k in out:
                tol.long_sum_close(out[k].cpu().numpy(), ref[k], rows)


def test_config1_layernorm_forward_fp32_full_size():
    """x[64,128,512] ~N(0,1), gamma=1+N(0,0.02), beta~N(0,0.02), eps=1e-5, seed 0."""
    torch.manual_seed(0)
    x = torch.randn(64, 128, 512)
    gamma = 1 + 0.02 * torch.randn(512)
    beta = 0.02 * torch.randn(512)
    y, mean, rstd = abi.layernorm_fwd(x.view(-1, 512).cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    ref = O.layernorm_act(x.view(-1, 512).numpy(), gamma.numpy(), beta.numpy(), None, 1e-5)
    check(y, ref["y"], "config 1 y")
    if R.available():   # the reference's own module on CPU, same inputs
        r = R.layernorm_act(x.view(-1, 512).numpy(), gamma.numpy(), beta.numpy(), None, 1e-5)
        tol.fp32_close_adjudicated(y.cpu().numpy(), r["y"], ref["y"])


def test_config2_layernorm_gelu_fwd_bwd_fp32_full_size():
    """x[32,1024,1024], dY same shape, exact-erf GELU, eps=1e-5: y, dX, dgamma, dbeta."""
    rows, D = 32 * 1024, 1024
    x, xn = make((rows, D), 0, torch.float32)
    dy, dyn = make((rows, D), 1, torch.float32)
    gamma, gn = make((D,), 2, torch.float32, 0.02, 1.0)
    beta, bn = make((D,), 3, torch.float32, 0.02)
    out = run_gpu("ln", x, gamma, beta, dy, 1e-5, abi.ACT_GELU)
    ref = O.layernorm_act(xn, gn, bn, dyn, 1e-5, O.ACT_GELU)
    check(out["y"], ref["y"], "config 2 y")
    check(out["dx"], ref["dx"], "config 2 dx")
    if R.available():
        # the reference's own modules on CPU, run in fp32 and again in fp64 (its autograd gives dgamma/dbeta in both)
        r = R.layernorm_act(xn, gn, bn, dyn, 1e-5, 1, compute=0)
        r64 = R.layernorm_act(xn, gn, bn, dyn, 1e-5, 1, compute=1)
        tol.fp32_close_adjudicated(out["y"].cpu().numpy(), r["y"], ref["y"])
        tol.fp32_close_adjudicated(out["dx"].cpu().numpy(), r["dx"], ref["dx"])
        # 32768-term sums: stated tolerance against fp64 or fp32 CPU, or closer to fp64 than fp32 CPU is;
        # the sqrt(n) allowance is not accepted here
        tol.long_sum_close(out["dgamma"].cpu().numpy(), r64["dgamma64"], rows, ref32=r["dgamma"], strict=True, label="cfg2 ln fp32 dgamma")
        tol.long_sum_close(out["dbeta"].cpu().numpy(), r64["dbeta64"], rows, ref32=r["dbeta"], strict=True, label="cfg2 ln fp32 dbeta")
        # the C restatement and the reference's fp64 run agree far inside the tolerance
        tol.fp32_close(ref["dgamma"], r64["dgamma64"], rtol=1e-9, atol=1e-7)
    else:
        tol.long_sum_close(out["dgamma"].cpu().numpy(), ref["dgamma"], rows)
        tol.long_sum_close(out["dbeta"].cpu().numpy(), ref["dbeta"], rows)
    # run-to-run determinism
    again = run_gpu("ln", x, gamma, beta, dy, 1e-5, abi.ACT_GELU)
    for k in ("y", "dx", "dgamma", "dbeta"):
        assert torch.equal(out[k], again[k]), k


def _device_inputs(kind, dtype, rows, D, seed):
    """Seeded N(0,1) activations made on the device (the full-size cases are too large to draw on the host)."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, D, device="cuda", generator=gen).to(dtype)
    dy = torch.randn(rows, D, device="cuda", generator=gen).to(dtype)
    gamma, gn = make((D,), 9, dtype, 0.02, 1.0)
    beta, bn = make((D,), 10, dtype, 0.02) if kind == "ln" else (None, None)
    return x, dy, gamma, gn, beta, bn


def _sampled_rows_check(kind, dtype, rows, D, act, eps, sample=48, blocks=8, label=None):
    """Full-size run on the GPU.  Rows are independent, so a scattered sample of them is checked against the
    oracle.  The parameter gradients are checked in two steps: whole-run sums == sum of the row blocks' sums
    (additivity, a consistency property between GPU results, so the natural-magnitude allowance applies), and
    one block of up to 16384 rows against the reference's own fp32 and fp64 CPU runs under the strict rule."""
    torch.cuda.empty_cache()                              # the largest case holds 69 GB of activations
    x, dy, gamma, gn, beta, bn = _device_inputs(kind, dtype, rows, D, 7)
    out = run_gpu(kind, x, gamma, beta, dy, eps, act)
    idx = torch.linspace(0, rows - 1, sample).long()
    xs, dys = x[idx.cuda()].float().cpu().numpy(), dy[idx.cuda()].float().cpu().numpy()
    ref = O.layernorm_act(xs, gn, bn, dys, eps, act) if kind == "ln" else O.rmsnorm_act(xs, gn, dys, eps, act)
    check(out["y"][idx.cuda()], ref["y"], "sampled y")
    check(out["dx"][idx.cuda()], ref["dx"], "sampled dx")
    # checksum of checksums: gradients of the whole = sum of gradients of the row blocks
    keys = ("dgamma", "dbeta") if kind == "ln" else ("dweight",)
    acc = {k: torch.zeros(D, dtype=torch.float64, device="cuda") for k in keys}
    step = rows // blocks
    for b in range(blocks):
        sl = slice(b * step, rows if b == blocks - 1 else (b + 1) * step)
        part = run_gpu(kind, x[sl], gamma, None if beta is None else beta, dy[sl], eps, act)
        for k in keys:
            acc[k] += part[k].double()
    for k in keys:
        tol.long_sum_close(out[k].cpu().numpy(), acc[k].cpu().numpy(), rows)
    # one block against the reference pins the blocks themselves (at most 16 Mi elements: the CPU runs take seconds)
    nb = max(1, min(step, 16384, (16 << 20) // D))
    part = run_gpu(kind, x[:nb], gamma, beta, dy[:nb], eps, act)
    xs, dys = x[:nb].float().cpu().numpy(), dy[:nb].float().cpu().numpy()
    name = label or f"cfg5 {kind} {'bf16' if dtype == torch.bfloat16 else 'fp32'} D={D} rows={rows}"
    if R.available():
        # the reference's modules in fp32 (the stated comparison) and in fp64 (the arbiter)
        r32 = R.layernorm_act(xs, gn, bn, dys, eps, act, compute=0) if kind == "ln" else R.rmsnorm_act(xs, gn, dys, eps, act, compute=0)
        r64 = R.layernorm_act(xs, gn, bn, dys, eps, act, compute=1) if kind == "ln" else R.rmsnorm_act(xs, gn, dys, eps, act, compute=1)
        for k in keys:
            tol.long_sum_close(part[k].cpu().numpy(), r64[k + "64"], nb, ref32=r32[k], strict=True, label=f"{name}: {k} of a {nb}-row block")
    else:
        nb = min(nb, 512)
        part = run_gpu(kind, x[:nb], gamma, beta, dy[:nb], eps, act)
        ref = O.layernorm_act(xs[:nb], gn, bn, dys[:nb], eps, act) if kind == "ln" else O.rmsnorm_act(xs[:nb], gn, dys[:nb], eps, act)
        for k in keys:
            tol.long_sum_close(part[k].cpu().numpy(), ref[k], nb)
    assert abi.device_status() == 0
    del x, dy, out, part
    torch.cuda.empty_cache()


def test_config3_rmsnorm_bf16_full_size():
    """x[16,4096,4096] bf16, weight=1+N(0,0.02), eps=1e-6, fwd + bwd."""
    _sampled_rows_check("rms", torch.bfloat16, 16 * 4096, 4096, abi.ACT_NONE, 1e-6)


@pytest.mark.parametrize("kind,act", [("ln", abi.ACT_GELU), ("rms", abi.ACT_SILU)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [768, 2048, 8192])
def test_config5_sweep_shapes_sampled(kind, act, dtype, D):
    """The whole-box sweep's widths at 2^16 rows per GPU (2^20 rows over 16 shards)."""
    _sampled_rows_check(kind, dtype, 1 << 16, D, act, 1e-5 if kind == "ln" else 1e-6, sample=24)


@pytest.mark.parametrize("kind,act,dtype", [("ln", abi.ACT_GELU, torch.float32), ("ln", abi.ACT_GELU, torch.bfloat16),
                                            ("rms", abi.ACT_SILU, torch.float32), ("rms", abi.ACT_SILU, torch.bfloat16)])
@pytest.mark.parametrize("D", [1024, 2048, 4096])
def test_config5_all_2p20_rows_on_one_gpu(kind, act, dtype, D):
    """The sweep at the row count the benchmark runs on one GPU: 2^20 rows (up to 69 GB of activations),
    64 row blocks for the additivity check."""
    _sampled_rows_check(kind, dtype, 1 << 20, D, act, 1e-5 if kind == "ln" else 1e-6, sample=64, blocks=64)


def test_no_affine_no_stats_and_empty():
    x, xn = make((17, 1024), 5, torch.float32)
    y, mean, rstd = abi.layernorm_fwd(x, None, None, 1e-5, abi.ACT_GELU, want_stats=False)
    assert mean is None and rstd is None
    check(y, O.layernorm_act(xn, None, None, None, 1e-5, O.ACT_GELU)["y"], "no affine y")
    y, rstd = abi.rmsnorm_fwd(x, None, 1e-6, abi.ACT_NONE)
    check(y, O.rmsnorm_act(xn, None, None, 1e-6)["y"], "no weight y")
    e = torch.empty(0, 1024, device="cuda")
    y, mean, rstd = abi.layernorm_fwd(e, None, None, 1e-5)
    assert y.shape == (0, 1024)
    dx, gb = abi.layernorm_bwd(e, e, None, None, mean, rstd, want_param_grads=True)
    assert dx.shape == (0, 1024) and float(gb.abs().sum()) == 0.0


def test_unaligned_views_take_the_any_width_path():
    base, bn = make((9 * 1024 + 1,), 6, torch.float32)
    x = base[1:].view(9, 1024)                       # 4-byte aligned only
    gamma, gn = make((1024,), 7, torch.float32, 0.02, 1.0)
    beta, bnn = make((1024,), 8, torch.float32, 0.02)
    assert x.data_ptr() % 16 != 0
    y, mean, rstd = abi.layernorm_fwd(x, gamma, beta, 1e-5, abi.ACT_SILU)
    ref = O.layernorm_act(bn[1:].reshape(9, 1024), gn, bnn, None, 1e-5, O.ACT_SILU)
    check(y, ref["y"], "unaligned y")


def test_no_kernel_gave_up_waiting():
    """The ring kernels bound every wait and report through the device status word."""
    x, _ = make((4096, 1024), 11, torch.float32)
    g, _ = make((1024,), 12, torch.float32, 0.02, 1.0)
    b, _ = make((1024,), 13, torch.float32, 0.02)
    y, mean, rstd = abi.layernorm_fwd(x, g, b, 1e-5, abi.ACT_GELU)
    abi.layernorm_bwd(x, x, g, b, mean, rstd, abi.ACT_GELU)
    torch.cuda.synchronize()
    assert abi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm_statistics_with_an_outlying_first_column_and_a_large_offset(dtype):
    """Rows whose first column is far from the rest, and rows with a mean far above their spread, are where
    a statistics shortcut (one-pass sums, a shift by a sampled column) would lose digits; the two-pass
    statistics must match the oracle there."""
    rows, D = 96, 1024
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(rows, D, generator=gen)
    x[:32] = x[:32] * 0.1 + 10.0              # mean = 100 x spread (fp32 input rounding alone costs 6e-6 on xhat)
    x[32:64, 0] = 5000.0                      # first column 5000 sigma away
    x[64:, 0] = -7.5
    x = x.to(dtype)
    g, gn = make((D,), 2, dtype, 0.02, 1.0); b, bn = make((D,), 3, dtype, 0.02)
    y, mean, rstd = abi.layernorm_fwd(x.cuda(), g, b, 1e-5, abi.ACT_NONE)
    ref = O.layernorm_act(x.float().numpy(), gn, bn, None, 1e-5, abi.ACT_NONE)
    np.testing.assert_allclose(mean.cpu().numpy(), ref["mean"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(rstd.cpu().numpy(), ref["rstd"], rtol=2e-5)
    if dtype == torch.float32:
        # y = xhat*gamma+beta with |xhat| up to 32 (the outlier itself): relative tolerance on that scale
        np.testing.assert_allclose(y.cpu().numpy(), ref["y"], rtol=2e-5, atol=2e-5)
    else:
        check(y, ref["y"], "y")


def test_reserved_sms_change_the_grid_not_the_results():
    """nb2_reserve_sms(n): the persistent kernels run on fewer CTAs; rows are independent, so y and dX keep
    their bits, and the parameter gradients (summed over a different number of partials) stay in tolerance."""
    rows, D = 20000, 1024
    x, xn = make((rows, D), 1, torch.float32); dy, dyn = make((rows, D), 2, torch.float32)
    g, gn = make((D,), 3, torch.float32, 0.02, 1.0); b, bn = make((D,), 4, torch.float32, 0.02)
    base = run_gpu("ln", x, g, b, dy, 1e-5, abi.ACT_GELU)
    L = abi.lib()
    before = L.nb2_reserve_sms(16)
    try:
        held = run_gpu("ln", x, g, b, dy, 1e-5, abi.ACT_GELU)
    finally:
        L.nb2_reserve_sms(before)
    assert torch.equal(base["y"], held["y"]) and torch.equal(base["dx"], held["dx"])
    ref = O.layernorm_act(xn, gn, bn, dyn, 1e-5, abi.ACT_GELU)
    tol.long_sum_close(held["dgamma"].cpu().numpy(), ref["dgamma"], rows)
    tol.long_sum_close(held["dbeta"].cpu().numpy(), ref["dbeta"], rows)
    assert abi.device_status() == 0


def test_reserved_sms_also_shrink_the_register_row_grids():
    """RMSNorm fp32 with rows under 16 KiB takes the register-row kernels in both directions; they honour the
    reservation as the ring kernels do (fewer CTAs, so fewer partials), with unchanged y and dX."""
    rows, D = 20000, 1024
    x, xn = make((rows, D), 1, torch.float32); dy, dyn = make((rows, D), 2, torch.float32)
    w, wn = make((D,), 3, torch.float32, 0.02, 1.0)
    L = abi.lib()
    code = abi.dtype_code(torch.float32)

    def bwd_partials():
        y, rstd = abi.rmsnorm_fwd(x, w, 1e-6, abi.ACT_SILU)
        dx = torch.empty_like(x)
        parts = torch.empty(abi.workspace_bytes(abi.WS_NORM_BWD, rows, D, code) // 4, device="cuda")
        import ctypes
        n = ctypes.c_int64(0)
        abi.check(L.nb2_rmsnorm_bwd(x.data_ptr(), dy.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), parts.data_ptr(),
                                    ctypes.byref(n), rows, D, code, abi.ACT_SILU, None))
        torch.cuda.synchronize()
        return y, dx, n.value

    y0, dx0, n0 = bwd_partials()
    before = L.nb2_reserve_sms(16)
    try:
        y1, dx1, n1 = bwd_partials()
    finally:
        L.nb2_reserve_sms(before)
    sms = L.nb2_sm_count()
    assert n0 == 2 * sms and n1 == 2 * (sms - 16), (n0, n1, sms)
    assert torch.equal(y0, y1) and torch.equal(dx0, dx1)
