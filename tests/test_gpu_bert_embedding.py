"""BERT embedding front end (gathers + LayerNorm eps 1e-12) fused: C ABI and C++ module."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from tests import tol
from tests.gpu_util import bits, check, make, to_dev
from thot_b200 import abi

pytestmark = pytest.mark.gpu


def test_golden_reference_module(golden_dir):
    z = np.load(golden_dir / "bert_embedding.npz")
    g = {k: z[k] for k in z.files}
    dev = lambda k: to_dev(g[k], torch.float32)  # noqa: E731
    ids = torch.from_numpy(g["ids"]).cuda()
    y, ssum, mean, rstd = abi.bert_embedding_ln_fwd(dev("word"), dev("pos"), dev("type"), ids, dev("gamma"), dev("beta"))
    tol.fp32_close(y.cpu().numpy(), g["y_f32"], rtol=2e-5, atol=2e-6)
    dword, dpos, dtype0, grads, _ = abi.bert_embedding_ln_bwd(ssum, dev("dy"), ids, dev("gamma"), mean, rstd, 50, pos_rows=16)
    np.testing.assert_allclose(dword.cpu().numpy(), g["dword_f64"], rtol=2e-5, atol=2e-4)
    np.testing.assert_allclose(dpos.cpu().numpy(), g["dpos_f64"], rtol=2e-5, atol=2e-4)
    np.testing.assert_allclose(dtype0.cpu().numpy(), g["dtype_f64"][0], rtol=2e-5, atol=2e-4)
    tol.long_sum_close(grads[0].cpu().numpy(), g["dgamma_f64"], 21, ref32=g["dgamma_f32"])
    tol.long_sum_close(grads[1].cpu().numpy(), g["dbeta_f64"], 21, ref32=g["dbeta_f32"])
    # int32 ids take the same path
    y32, *_ = abi.bert_embedding_ln_fwd(dev("word"), dev("pos"), dev("type"), ids.int(), dev("gamma"), dev("beta"))
    assert torch.equal(y, y32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,D,B,S,use_pos,use_type", [(30522, 768, 8, 128, True, True), (1000, 1024, 3, 77, True, False),
                                                         (64, 100, 2, 9, False, True), (500, 4096, 2, 33, True, True)])
def test_against_oracle(dtype, vocab, D, B, S, use_pos, use_type):
    eps = 1e-5                     # a generic eps keeps bf16 outputs O(1); the reference's 1e-12 is in the golden test
    word, wn = make((vocab, D), 1, dtype, 0.5)
    pos, pn = make((max(S, 16), D), 2, dtype, 0.5) if use_pos else (None, None)
    typ, tn = make((2, D), 3, dtype, 0.5) if use_type else (None, None)
    gamma, gn = make((D,), 4, dtype, 0.02, 1.0); beta, bn = make((D,), 5, dtype, 0.02)
    gen = torch.Generator().manual_seed(6)
    ids = torch.randint(0, vocab, (B, S), generator=gen)
    dy, dyn = make((B, S, D), 7, dtype)
    y, ssum, mean, rstd = abi.bert_embedding_ln_fwd(word, pos, typ, ids.cuda(), gamma, beta, eps)
    ref = O.bert_embedding(wn, pn, tn, gn, bn, ids.numpy(), dyn, eps, bf16=dtype == torch.bfloat16)
    if dtype == torch.float32:
        assert np.array_equal(ssum.cpu().numpy(), ref["sum"])
    else:
        assert np.array_equal(bits(ssum), tol.to_bf16_bits(ref["sum"]))
    check(y.reshape(B * S, D), ref["y"].reshape(B * S, D), "y")
    dword, dpos, dtype0, grads, dsum = abi.bert_embedding_ln_bwd(ssum, dy, ids.cuda(), gamma, mean, rstd, vocab,
                                                                pos_rows=pos.shape[0] if use_pos else 0, want_type=use_type)
    # stage 1: the gradient of the sum (LayerNorm backward), a tensor of the activation dtype
    check(dsum, ref["dsum"] if dtype == torch.float32 else O.layernorm_act(ref["sum"], gn, bn, dyn.reshape(B * S, D), eps)["dx"], "dsum")
    # stage 2: the table gradients are sums of rows of THAT tensor (fp32 accumulation, one rounding)
    ds = dsum.float().cpu().numpy().astype(np.float64)
    check(dword, O._scatter_rows(ds, ids.numpy().reshape(-1), vocab), "dword")
    if use_pos:
        full = np.zeros((pos.shape[0], D)); full[:S] = ds.reshape(B, S, D).sum(axis=0)
        check(dpos, full, "dpos")
    if use_type:
        if dtype == torch.float32:
            tol.long_sum_close(dtype0.cpu().numpy(), ds.sum(axis=0), B * S)       # a B*S-term fp32 sum
        else:
            tol.bf16_ulp_close(bits(dtype0), ds.sum(axis=0))
    tol.long_sum_close(grads[0].cpu().numpy(), ref["dgamma"], B * S)
    tol.long_sum_close(grads[1].cpu().numpy(), ref["dbeta"], B * S)


def test_bad_ids_and_module_names():
    word, _ = make((10, 64), 1, torch.float32)
    g, _ = make((64,), 2, torch.float32, 0.02, 1.0); b, _ = make((64,), 3, torch.float32, 0.02)
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    ids = torch.tensor([[1, 99, 3]], device="cuda")
    y, *_ = abi.bert_embedding_ln_fwd(word, None, None, ids, g, b, 1e-5, status=status)
    assert status[0].item() == 1 and status[1].item() == 1 and torch.isfinite(y).all()
    from thot_b200 import _nott_b200_host as host
    ids = torch.randint(0, 40, (2, 5), device="cuda")
    dy = torch.randn(2, 5, 32, device="cuda")
    names, out = host.bert_embedding_module_step(32, 40, 2, 8, ids, dy, [])
    assert names == ["word_embeddings.weight", "token_type_embeddings.weight", "position_embeddings.weight",
                     "layer_norm.weight", "layer_norm.bias"]
    assert out[0].shape == (2, 5, 32) and all(t is not None for t in out[1:])
    assert not out[2][1].any() and not out[3][5:].any()      # type row 1 and positions >= S get no gradient


def test_ready_made_embeddings_golden_through_the_module(golden_dir):
    """BertEmbedding fed [B, S, D] embeddings instead of ids (bert.hpp:164-171): position and type rows are
    added and the sum is LayerNorm'ed; the C++ drop-in module against the reference module's own outputs."""
    from thot_b200 import _nott_b200_host as host
    z = np.load(golden_dir / "bert_embedding_float_input.npz")
    g = {k: z[k] for k in z.files}
    B, S, D = g["input"].shape
    dev = lambda k: to_dev(g[k], torch.float32)  # noqa: E731
    word = torch.zeros(4, D, device="cuda")
    # parameter order of the module: word, token type, position, layer_norm.weight, layer_norm.bias
    names, out = host.bert_embedding_module_step(D, 4, g["type"].shape[0], g["pos"].shape[0], dev("input"), dev("dy"),
                                                 [word, dev("type"), dev("pos"), dev("gamma"), dev("beta")])
    y, dword, dtype, dpos, dgamma, dbeta, dinput = out
    tol.fp32_close(y.cpu().numpy(), g["y_f32"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(dinput.cpu().numpy(), g["dinput_f64"], rtol=2e-5, atol=2e-4)
    np.testing.assert_allclose(dpos.cpu().numpy(), g["dpos_f64"], rtol=2e-5, atol=2e-4)
    np.testing.assert_allclose(dtype.cpu().numpy(), g["dtype_f64"], rtol=2e-5, atol=2e-4)
    tol.long_sum_close(dgamma.cpu().numpy(), g["dgamma_f64"], B * S, ref32=g["dgamma_f32"])
    tol.long_sum_close(dbeta.cpu().numpy(), g["dbeta_f64"], B * S, ref32=g["dbeta_f32"])
    assert float(dword.abs().sum()) == 0.0                  # the word table is not part of this branch
    with pytest.raises(Exception, match="expected last dimension"):
        host.bert_embedding_module_step(D, 4, 2, 16, torch.zeros(2, 3, D + 1, device="cuda"), torch.zeros(2, 3, D + 1, device="cuda"), [])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,B,S,use_pos,use_type", [(768, 8, 128, True, True), (1024, 3, 77, True, False), (100, 2, 9, False, True),
                                                    (96, 2, 5, False, False)])
def test_ready_made_embeddings_against_oracle(dtype, D, B, S, use_pos, use_type):
    eps = 1e-5
    inp, inn = make((B, S, D), 1, dtype, 0.5)
    pos, pn = make((max(S, 16), D), 2, dtype, 0.5) if use_pos else (None, None)
    typ, tn = make((2, D), 3, dtype, 0.5) if use_type else (None, None)
    gamma, gn = make((D,), 4, dtype, 0.02, 1.0); beta, bn = make((D,), 5, dtype, 0.02)
    dy, dyn = make((B, S, D), 7, dtype)
    L = abi.lib()
    import ctypes
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())  # noqa: E731
    code = abi.dtype_code(dtype)
    y = torch.empty_like(inp); ssum = torch.empty(B * S, D, dtype=dtype, device="cuda")
    mean = torch.empty(B * S, device="cuda"); rstd = torch.empty(B * S, device="cuda")
    abi.check(L.nb2_bert_embedding_ln_fwd(P(inp), P(pos), P(typ), None, P(gamma), P(beta), P(ssum), P(y), P(mean), P(rstd),
                                          B, S, 1, D, eps, code, abi.I64, None, None))
    ref = O.bert_embedding(inn, pn, tn, gn, bn, None, dyn, eps, bf16=dtype == torch.bfloat16)
    if dtype == torch.float32:
        assert np.array_equal(ssum.cpu().numpy(), ref["sum"])
    else:
        assert np.array_equal(bits(ssum), tol.to_bf16_bits(ref["sum"]))
    check(y.reshape(B * S, D), ref["y"].reshape(B * S, D), "y")
    dsum = torch.empty_like(ssum)
    pos_rows = pos.shape[0] if use_pos else 0
    dpos = torch.empty(pos_rows, D, dtype=dtype, device="cuda") if use_pos else None
    dtype0 = torch.empty(D, dtype=dtype, device="cuda") if use_type else None
    grads = torch.empty(2, D, device="cuda")
    ws_bytes = abi.workspace_bytes(abi.WS_BERT_EMBEDDING_BWD, (B << 32) | S, ((B * S) << 32) | D, code)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    abi.check(L.nb2_bert_embedding_ln_bwd(P(ssum), P(dy), None, P(gamma), P(mean), P(rstd), P(dsum), None, P(dpos), pos_rows,
                                          P(dtype0), P(grads), B, S, B * S, D, code, abi.I64, P(ws), ws_bytes, None))
    check(dsum, ref["dsum"] if dtype == torch.float32 else O.layernorm_act(ref["sum"], gn, bn, dyn.reshape(B * S, D), eps)["dx"], "dsum")
    ds = dsum.float().cpu().numpy().astype(np.float64)
    if use_pos:
        full = np.zeros((pos_rows, D)); full[:S] = ds.reshape(B, S, D).sum(axis=0)
        check(dpos, full, "dpos")
    if use_type:
        if dtype == torch.float32:
            tol.long_sum_close(dtype0.cpu().numpy(), ds.sum(axis=0), B * S)
        else:
            tol.bf16_ulp_close(bits(dtype0), ds.sum(axis=0))
    tol.long_sum_close(grads[0].cpu().numpy(), ref["dgamma"], B * S)
    tol.long_sum_close(grads[1].cpu().numpy(), ref["dbeta"], B * S)
    assert abi.device_status() == 0
