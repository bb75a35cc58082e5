"""Row sharding of the norm path across the GPUs of one box.

Rows (batch x sequence) are independent, so forward and dX need no
communication; the only exchange is one sum-allreduce of the [2, D]
(LayerNorm: dgamma | dbeta) or [D] (RMSNorm: dweight) fp32 gradients, issued on
the compute stream right after the partial reduce.  One process per GPU,
torch.distributed for the plumbing (NCCL over NVLink on GPUs, gloo in CPU tests).
The reference itself is single-device (src/core.hpp:1706-1708 pins cuda:0).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def row_shard(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, even split: (first row, row count) of `rank`.  The first
    `rows % world` ranks hold one extra row; a rank may hold zero rows."""
    if world <= 0 or not 0 <= rank < world or rows < 0:
        raise ValueError(f"bad shard request rows={rows} world={world} rank={rank}")
    base, extra = divmod(rows, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def allreduce_param_grads(grads: torch.Tensor, group=None) -> torch.Tensor:
    """In-place SUM over ranks of the fp32 affine-parameter gradients.  A no-op
    when torch.distributed is not initialised or the world is one rank."""
    if grads.dtype != torch.float32:
        raise TypeError("affine-parameter gradients are exchanged in fp32")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(grads, op=dist.ReduceOp.SUM, group=group)
    return grads


class ShardedNormStep:
    """Forward + backward of LayerNorm/RMSNorm (+activation) on this rank's row
    shard, then the allreduce.  `kind` is "ln" or "rms"."""

    def __init__(self, kind: str, eps: float, act: int, group=None):
        if kind not in ("ln", "rms"):
            raise ValueError(kind)
        self.kind, self.eps, self.act, self.group = kind, eps, act, group

    def __call__(self, x, dy, gamma, beta=None):
        from . import abi

        if self.kind == "ln":
            y, mean, rstd = abi.layernorm_fwd(x, gamma, beta, self.eps, self.act)
            dx, grads = abi.layernorm_bwd(x, dy, gamma, beta, mean, rstd, self.act)
        else:
            y, rstd = abi.rmsnorm_fwd(x, gamma, self.eps, self.act)
            dx, grads = abi.rmsnorm_bwd(x, dy, gamma, rstd, self.act)
        allreduce_param_grads(grads, self.group)
        return y, dx, grads
