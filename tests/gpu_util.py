"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

from tests import tol


def make(shape, seed, dtype, scale=1.0, shift=0.0):
    """Seeded CPU fp32 normal values, rounded to `dtype`; returns (device tensor, fp32 numpy of the
    values the device tensor holds)."""
    gen = torch.Generator().manual_seed(seed)
    t = (torch.randn(*shape, generator=gen) * scale + shift).to(dtype)
    return t.cuda(), t.to(torch.float32).numpy()


def to_dev(a: np.ndarray, dtype):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(dtype).cuda()


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def check(got: torch.Tensor, ref, what=""):
    """fp32: 1e-5 rel / 1e-6 abs.  bf16: 2 ulp of the reference rounded to bf16."""
    try:
        if got.dtype == torch.bfloat16:
            tol.bf16_ulp_close(bits(got), np.asarray(ref, np.float32))
        else:
            tol.fp32_close(got.cpu().numpy(), ref)
    except AssertionError as e:
        raise AssertionError(f"{what}: {e}") from None
