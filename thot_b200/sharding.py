"""Row sharding of the norm path across the GPUs of one box: host-side helpers.

Rows (batch x sequence) are independent, so forward and dX need no
communication; the only exchange is one sum over ranks of the [2, D]
(LayerNorm: dgamma | dbeta) or [D] (RMSNorm: dweight) fp32 gradients.  On GPUs
that exchange is the C step driver's (nb2_step_run / nb2_grad_exchange_* in
include/nott_b200.h, wrapped by thot_b200.abi.Comm and NormStep), which calls
NCCL or the library's own peer-store kernels itself.  This module holds what
needs no GPU: the row partition, a layout check that turns a rank with another
D into an error instead of a hung collective, and the same exchange over a
torch.distributed group (gloo in the CPU tests) with a deadline.
The reference itself is single-device (src/core.hpp:1706-1708 pins cuda:0).
"""
from __future__ import annotations

from datetime import timedelta
from typing import Optional, Tuple

import torch
import torch.distributed as dist


class ExchangeError(RuntimeError):
    """The gradient exchange failed or did not finish before its deadline."""


def row_shard(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, even split: (first row, row count) of `rank`.  The first
    `rows % world` ranks hold one extra row; a rank may hold zero rows."""
    if world <= 0 or not 0 <= rank < world or rows < 0:
        raise ValueError(f"bad shard request rows={rows} world={world} rank={rank}")
    base, extra = divmod(rows, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def _active(group) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def check_layout(ncols: int, norm: str, dtype_code: int, group=None, timeout_s: float = 30.0) -> None:
    """Every rank must exchange a gradient vector of the same length for the same norm.  Called once
    when a sharded step is set up: a rank configured with another D would otherwise leave the sum
    over ranks waiting for bytes that never come.  Raises ExchangeError naming the ranks that differ."""
    if not _active(group):
        return
    world = dist.get_world_size(group)
    mine = torch.tensor([int(ncols), 0 if norm == "ln" else 1, int(dtype_code)], dtype=torch.int64)
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    work = dist.all_gather(gathered, mine, group=group, async_op=True)
    _wait(work, timeout_s, "layout check")
    layouts = [tuple(int(v) for v in t) for t in gathered]
    if any(l != layouts[0] for l in layouts):
        raise ExchangeError(f"ranks disagree on the gradient layout (ncols, norm, dtype): {layouts}")


def _wait(work, timeout_s: Optional[float], what: str) -> None:
    try:
        if timeout_s is None:
            work.wait()
        else:
            ok = work.wait(timedelta(seconds=timeout_s))
            if ok is False:
                raise ExchangeError(f"{what} did not finish within {timeout_s} s")
    except ExchangeError:
        raise
    except RuntimeError as exc:          # gloo reports a timeout or a dead peer as RuntimeError
        raise ExchangeError(f"{what} failed: {exc}") from exc


def allreduce_param_grads(grads: torch.Tensor, group=None, timeout_s: Optional[float] = None) -> torch.Tensor:
    """In-place SUM over ranks of the fp32 affine-parameter gradients.  A no-op when
    torch.distributed is not initialised or the world is one rank.  With `timeout_s`, a peer that
    never joins makes this raise ExchangeError after the deadline instead of blocking."""
    if grads.dtype != torch.float32:
        raise TypeError("affine-parameter gradients are exchanged in fp32")
    if _active(group):
        work = dist.all_reduce(grads, op=dist.ReduceOp.SUM, group=group, async_op=True)
        _wait(work, timeout_s, "gradient allreduce")
    return grads
