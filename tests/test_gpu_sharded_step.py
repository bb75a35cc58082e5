"""The C step driver (nb2_step_run) and the gradient exchange (nb2_grad_exchange_begin/end) through the
C ABI.  On one GPU the communicator has one rank: the NCCL form degenerates to the plain partial reduce and
the peer form runs its two kernels (store into the rank's own slot, collect) for real.  With two or more
GPUs a child process per GPU checks the sum over ranks against the unsharded oracle."""
from __future__ import annotations

import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import check, make
from thot_b200 import abi

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("exchange", [abi.EXCHANGE_NCCL, abi.EXCHANGE_PEER])
@pytest.mark.parametrize("kind,dtype,rows,D,act", [("ln", torch.float32, 4100, 1024, abi.ACT_GELU),
                                                   ("rms", torch.bfloat16, 3000, 2048, abi.ACT_SILU),
                                                   ("ln", torch.float32, 37, 1000, abi.ACT_NONE),      # any-width path, ncols % 32 != 0
                                                   ("rms", torch.float32, 50, 7, abi.ACT_GELU)])
def test_step_driver_matches_the_separate_calls_and_the_oracle(exchange, kind, dtype, rows, D, act):
    eps = 1e-5 if kind == "ln" else 1e-6
    x, xn = make((rows, D), 1, dtype); dy, dyn = make((rows, D), 2, dtype)
    g, gn = make((D,), 3, dtype, 0.02, 1.0)
    b, bn = make((D,), 4, dtype, 0.02) if kind == "ln" else (None, None)
    comm = abi.Comm(None, 0, 1, exchange, max_cols=2 * D)
    step = abi.NormStep(comm, kind, rows, D, dtype, act, eps)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    ncols = (2 if kind == "ln" else 1) * D
    grads = [torch.full((ncols,), float("nan"), device="cuda") for _ in range(2)]
    for k in range(3):                                    # three steps: both slot parities of the peer form are reused
        step.run(x, dy, g, b, y, dx, grads[k & 1])
    step.finish()
    comm.wait(10.0)
    torch.cuda.synchronize()
    assert torch.equal(grads[0], grads[1])                # same inputs every step, deterministic sums
    if kind == "ln":
        y0, mean, rstd = abi.layernorm_fwd(x, g, b, eps, act)
        dx0, gb0 = abi.layernorm_bwd(x, dy, g, b, mean, rstd, act)
        ref = O.layernorm_act(xn, gn, bn, dyn, eps, act)
        keys = ("dgamma", "dbeta")
    else:
        y0, rstd = abi.rmsnorm_fwd(x, g, eps, act)
        dx0, gb0 = abi.rmsnorm_bwd(x, dy, g, rstd, act)
        ref = O.rmsnorm_act(xn, gn, dyn, eps, act)
        keys = ("dweight",)
    assert torch.equal(y, y0) and torch.equal(dx, dx0)
    assert torch.equal(grads[0], gb0.reshape(-1))         # one rank: the exchange adds nothing
    check(y, ref["y"], "y"); check(dx, ref["dx"], "dx")
    got = grads[0].cpu().numpy().reshape(len(keys), D)
    for i, k in enumerate(keys):
        tol.long_sum_close(got[i], ref[k], rows)
    step.close(); comm.close()
    assert abi.device_status() == 0


def test_exchange_of_a_single_vector_and_argument_checks():
    comm = abi.Comm(None, 0, 1, abi.EXCHANGE_PEER, max_cols=4096)
    v = torch.randn(4096, device="cuda")
    keep = v.clone()
    comm.allreduce_(v)
    torch.cuda.synchronize()
    assert torch.equal(v, keep)
    big = torch.zeros(8192, device="cuda")
    with pytest.raises(abi.Nb2Error, match="max_cols"):
        comm.exchange_begin(big, 1, big)
    comm.exchange_begin(keep, 1, v)
    with pytest.raises(abi.Nb2Error, match="still outstanding"):
        comm.exchange_begin(keep, 1, v)                   # the same buffer twice in a row without ending the first
    w = torch.zeros_like(v)
    comm.exchange_begin(keep * 2, 1, w)                   # another buffer: the launch also completes the first exchange
    comm.exchange_end()
    torch.cuda.synchronize()
    assert torch.equal(v, keep) and torch.equal(w, keep * 2)
    comm.close()
    with pytest.raises(abi.Nb2Error):
        abi.Comm(None, 3, 2, abi.EXCHANGE_NCCL)            # rank outside the world


def test_peer_wait_gives_up_and_reports_instead_of_hanging():
    """The collect kernel's wait on a flag no rank publishes runs out after its limit (about a millisecond
    here), the kernel returns by itself, the status word carries code 4 and the context stays usable."""
    comm = abi.Comm(None, 0, 1, abi.EXCHANGE_PEER, max_cols=64)
    assert abi.device_status() == 0
    abi.check(abi.lib().nb2_selftest_peer_wait(comm.handle, 2_000_000, None))
    torch.cuda.synchronize()
    with pytest.raises(abi.Nb2Error) as e:
        abi.device_status()
    assert e.value.status == -6 and "code 4" in str(e.value)
    assert abi.device_status() == 0                        # cleared by the read above
    v = torch.ones(64, device="cuda")
    comm.allreduce_(v)                                     # the communicator still works
    torch.cuda.synchronize()
    assert torch.equal(v, torch.ones(64, device="cuda"))
    comm.close()


@pytest.mark.parametrize("rows,chunk", [(1000, 128), (77, 1000)])
def test_rmsnorm_host_step_matches_device_path(rows, chunk):
    D = 2048
    gen = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, D, generator=gen).bfloat16().pin_memory()
    dy = torch.randn(rows, D, generator=gen).bfloat16().pin_memory()
    w = (1 + 0.02 * torch.randn(D, generator=gen)).bfloat16()
    y = torch.empty_like(x).pin_memory(); dx = torch.empty_like(x).pin_memory()
    dw = torch.empty(D).pin_memory()
    hs = abi.HostStep(rows, D, torch.bfloat16, chunk)
    for _ in range(2):
        hs.step_rms(x, dy, w, y, dx, dw, 1e-6, abi.ACT_SILU)
    hs.close()
    yd, rstd = abi.rmsnorm_fwd(x.cuda(), w.cuda(), 1e-6, abi.ACT_SILU)
    dxd, dwd = abi.rmsnorm_bwd(x.cuda(), dy.cuda(), w.cuda(), rstd, abi.ACT_SILU)
    assert torch.equal(y, yd.cpu()) and torch.equal(dx, dxd.cpu())
    ref = O.rmsnorm_act(x.float().numpy(), w.float().numpy(), dy.float().numpy(), 1e-6, O.ACT_SILU)
    tol.long_sum_close(dw.numpy(), ref["dweight"], rows)
    tol.fp32_close(dw.numpy(), dwd.cpu().numpy(), rtol=1e-5, atol=1e-5)


# ---- two or more GPUs: one child process per GPU
_CHILD = r"""
import os, sys, json
sys.path.insert(0, os.environ["NB2_ROOT"])
import numpy as np, torch, torch.distributed as dist
from thot_b200 import abi
from thot_b200.sharding import row_shard
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)      # host-side plumbing only
box = [abi.comm_unique_id() if rank == 0 else None]
dist.broadcast_object_list(box, src=0)
mode = int(os.environ["NB2_EXCHANGE"])
rows, D = 4099, 1024
gen = torch.Generator().manual_seed(5)
x = torch.randn(rows, D, generator=gen); dy = torch.randn(rows, D, generator=gen)
g = 1 + 0.02 * torch.randn(D, generator=gen); b = 0.02 * torch.randn(D, generator=gen)
start, count = row_shard(rows, world, rank)
comm = abi.Comm(box[0], rank, world, mode, max_cols=2 * D)
step = abi.NormStep(comm, "ln", count, D, torch.float32, abi.ACT_GELU, 1e-5)
xs, dys = x[start:start + count].cuda(), dy[start:start + count].cuda()
y, dx = torch.empty_like(xs), torch.empty_like(xs)
grads = [torch.zeros(2 * D, device="cuda") for _ in range(2)]
for k in range(4):
    step.run(xs, dys, g.cuda(), b.cuda(), y, dx, grads[k & 1])
step.finish()
comm.wait(20.0)
torch.cuda.synchronize()
status = abi.device_status()
out = {"rank": rank, "status": status, "same": bool(torch.equal(grads[0], grads[1]))}
np.save(os.path.join(os.environ["NB2_OUT"], f"grads{rank}.npy"), grads[1].cpu().numpy())
np.save(os.path.join(os.environ["NB2_OUT"], f"dx{rank}.npy"), dx.cpu().numpy())
json.dump(out, open(os.path.join(os.environ["NB2_OUT"], f"r{rank}.json"), "w"))
step.close(); comm.close()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("exchange", [abi.EXCHANGE_NCCL, abi.EXCHANGE_PEER])
def test_two_ranks_sum_to_the_unsharded_gradients(tmp_path, exchange):
    world = min(torch.cuda.device_count(), 2)
    if world < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NB2_ROOT=str(ROOT), NB2_OUT=str(tmp_path), NB2_EXCHANGE=str(exchange), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env))
    for p in procs:
        assert p.wait(timeout=300) == 0
    rows, D = 4099, 1024
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(rows, D, generator=gen); dy = torch.randn(rows, D, generator=gen)
    g = 1 + 0.02 * torch.randn(D, generator=gen); b = 0.02 * torch.randn(D, generator=gen)
    ref = O.layernorm_act(x.numpy(), g.numpy(), b.numpy(), dy.numpy(), 1e-5, O.ACT_GELU)
    got = [np.load(tmp_path / f"grads{r}.npy") for r in range(world)]
    if exchange == abi.EXCHANGE_PEER:
        assert np.array_equal(got[0], got[1])              # every rank adds the same slots in the same order
    for r in range(world):
        tol.long_sum_close(got[r][:D], ref["dgamma"], rows)
        tol.long_sum_close(got[r][D:], ref["dbeta"], rows)
    dx = np.concatenate([np.load(tmp_path / f"dx{r}.npy") for r in range(world)])
    tol.fp32_close(dx, ref["dx"])


@pytest.mark.parametrize("exchange", [abi.EXCHANGE_NCCL, abi.EXCHANGE_PEER])
def test_cpp_step_driver_classes(exchange):
    """Nott::B200::Communicator / ShardedNormStep (the C++ wrappers over nb2_comm / nb2_step) give the same bits as
    the separate ABI calls."""
    from thot_b200 import _nott_b200_host as host
    rows, D = 2000, 1024
    x, _ = make((rows, D), 1, torch.float32); dy, _ = make((rows, D), 2, torch.float32)
    g, _ = make((D,), 3, torch.float32, 0.02, 1.0); b, _ = make((D,), 4, torch.float32, 0.02)
    y, dx, g0, g1 = host.sharded_norm_steps(False, exchange, x, dy, g, b, 7, 1e-5, 3)       # 7 = Nott::Activation::Type::GeLU
    y0, mean, rstd = abi.layernorm_fwd(x, g, b, 1e-5, abi.ACT_GELU)
    dx0, gb0 = abi.layernorm_bwd(x, dy, g, b, mean, rstd, abi.ACT_GELU)
    assert torch.equal(y, y0) and torch.equal(dx, dx0)
    assert torch.equal(g0, gb0.reshape(-1)) and torch.equal(g1, gb0.reshape(-1))
    w, _ = make((D,), 5, torch.bfloat16, 0.02, 1.0)
    xb, dyb = x.bfloat16(), dy.bfloat16()
    y, dx, g0, g1 = host.sharded_norm_steps(True, exchange, xb, dyb, w, None, 6, 1e-6, 2)   # 6 = SiLU
    yr, rstd = abi.rmsnorm_fwd(xb, w, 1e-6, abi.ACT_SILU)
    dxr, dw = abi.rmsnorm_bwd(xb, dyb, w, rstd, abi.ACT_SILU)
    assert torch.equal(y, yr) and torch.equal(dx, dxr) and torch.equal(g1, dw) and torch.equal(g0, dw)


@pytest.mark.parametrize("exchange", [abi.EXCHANGE_NCCL, abi.EXCHANGE_PEER])
def test_a_rank_without_rows_contributes_zeros(exchange):
    """More ranks than rows: a rank whose shard is empty still takes part in the exchange, with zero sums."""
    D = 256
    comm = abi.Comm(None, 0, 1, exchange, max_cols=2 * D)
    step = abi.NormStep(comm, "ln", 0, D, torch.float32, abi.ACT_GELU, 1e-5)
    e = torch.empty(0, D, device="cuda")
    g = torch.ones(D, device="cuda"); b = torch.zeros(D, device="cuda")
    grads = [torch.full((2 * D,), float("nan"), device="cuda") for _ in range(2)]
    for k in range(2):
        step.run(e, e, g, b, e, e, grads[k])
    step.finish()
    torch.cuda.synchronize()
    assert float(grads[0].abs().sum()) == 0.0 and float(grads[1].abs().sum()) == 0.0
    step.close(); comm.close()
    assert abi.device_status() == 0


@pytest.mark.parametrize("world", [2, 5, 8, 16])
def test_peer_exchange_with_many_ranks_on_one_gpu(world):
    """The peer exchange with up to 16 ranks' worth of data on one GPU: `world` linked communicators whose "peer"
    buffers are all local.  Every rank's begin of a step is issued before any rank's begin of the next, so each
    launch's collect phase finds the previous step already stored by everyone.  Every rank must end up with the same
    bits: the fp64 sum of the ranks' fp32 sums in rank order, rounded once."""
    ncols, parts = 2 * 1024 + 8, 37                       # a column count that is not a multiple of the 32-column CTA tile
    comms = abi.comm_group(world, ncols)
    gen = torch.Generator(device="cuda").manual_seed(world)
    steps = 3
    grads = [[torch.full((ncols,), float("nan"), device="cuda") for _ in range(2)] for _ in range(world)]
    want = []
    for k in range(steps):
        per_rank = []
        for r, c in enumerate(comms):
            p = torch.randn(parts, ncols, device="cuda", generator=gen)
            per_rank.append(p.double().sum(0).float())    # what the partial reduce leaves on rank r (fp64 sum, rounded)
            c.exchange_begin(p, parts, grads[r][k & 1])
        total = torch.zeros(ncols, dtype=torch.float64, device="cuda")
        for v in per_rank:                                # rank order
            total += v.double()
        want.append(total.float())
    for c in comms:
        c.exchange_end()
    torch.cuda.synchronize()
    assert abi.device_status() == 0
    for r in range(world):
        assert torch.equal(grads[r][(steps - 1) & 1], want[steps - 1]), f"rank {r}, last step"
        assert torch.equal(grads[r][(steps - 2) & 1], want[steps - 2]), f"rank {r}, the step before"
    for c in comms:
        c.close()
