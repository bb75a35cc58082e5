"""The norm kernels inside a CUDA graph: the reference records whole training steps into CUDA
graphs (src/core.hpp:3856-3879), so every launch must be capturable (current stream, no
synchronisation, no allocation inside the library) and replay must reproduce the eager result."""
from __future__ import annotations

import ctypes

import pytest
import torch

from tests.gpu_util import make
from thot_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,D", [(torch.float32, 1024), (torch.bfloat16, 4096), (torch.float32, 513)])
def test_forward_backward_reduce_replay_matches_eager(dtype, D):
    rows = 4096
    x, _ = make((rows, D), 1, dtype); dy, _ = make((rows, D), 2, dtype)
    g, _ = make((D,), 3, dtype, 0.02, 1.0); b, _ = make((D,), 4, dtype, 0.02)
    code = abi.dtype_code(dtype)
    # eager result (also the warm-up: first-use set-up such as shared-memory opt-in happens here)
    y0, mean0, rstd0 = abi.layernorm_fwd(x, g, b, 1e-5, abi.ACT_GELU)
    dx0, gr0 = abi.layernorm_bwd(x, dy, g, b, mean0, rstd0, abi.ACT_GELU)
    # static buffers for the graph
    y = torch.empty_like(x); dx = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda"); rstd = torch.empty(rows, device="cuda")
    partials = torch.empty(abi.workspace_bytes(abi.WS_NORM_BWD, rows, D, code) // 4, device="cuda")
    grads = torch.empty(2, D, device="cuda")
    L = abi.lib()
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    n = ctypes.c_int64(0)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        abi.check(L.nb2_layernorm_fwd(P(x), P(g), P(b), P(y), P(mean), P(rstd), rows, D, 1e-5, code, abi.ACT_GELU, st))
        abi.check(L.nb2_layernorm_bwd(P(x), P(dy), P(g), P(b), P(mean), P(rstd), P(dx), P(partials), ctypes.byref(n), rows, D,
                                      code, abi.ACT_GELU, st))
        abi.check(L.nb2_colreduce_partials(P(partials), n.value, 2 * D, P(grads), st))
    for t in (y, dx, grads):
        t.fill_(float("nan"))
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, y0) and torch.equal(dx, dx0) and torch.equal(grads, gr0)
    assert abi.device_status() == 0


def test_bert_backward_with_its_side_stream_is_capturable():
    """The BERT front-end backward sorts the ids on a side stream beside the LayerNorm backward;
    a capture must follow that fork and join, and the replay must reproduce the eager gradients."""
    B, S, D, vocab = 8, 64, 768, 1000
    dtype = torch.bfloat16
    ssum, _ = make((B * S, D), 1, dtype); dy, _ = make((B, S, D), 2, dtype)
    g, _ = make((D,), 3, dtype, 0.02, 1.0)
    ids = torch.randint(0, vocab, (B, S), generator=torch.Generator().manual_seed(4)).cuda()
    mean = ssum.float().mean(-1); rstd = torch.rsqrt(ssum.float().var(-1, unbiased=False) + 1e-5)
    dword0, dpos0, dtype00, grads0, dsum0 = abi.bert_embedding_ln_bwd(ssum, dy, ids, g, mean, rstd, vocab, pos_rows=S)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = abi.bert_embedding_ln_bwd(ssum, dy, ids, g, mean, rstd, vocab, pos_rows=S)
    for t in out:
        t.fill_(float("nan"))
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    for got, want in zip(out, (dword0, dpos0, dtype00, grads0, dsum0)):
        assert torch.equal(got, want)
    assert abi.device_status() == 0
