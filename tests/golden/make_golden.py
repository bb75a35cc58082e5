"""Regenerates tests/golden/*.npz from the reference's own modules on CPU.

Runs oracle/_ref/libnott_ref.so (oracle/ref_harness.cpp compiled against the
reference's headers and libtorch) on small seeded inputs and stores inputs and
outputs, in fp32 and fp64 module precision.  Needs the reference checkout to
build the harness; the committed .npz files are what the tests read.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref, reference as R  # noqa: E402

OUT = Path(__file__).resolve().parent


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


def randn(gen, *shape, scale=1.0, shift=0.0, bf16=False):
    a = (torch.randn(*shape, generator=gen) * scale + shift).numpy().astype(np.float32)
    return bf16_round(a) if bf16 else a


def norm_case(kind, seed, rows, D, eps, act, affine=True, bf16=False):
    gen = torch.Generator().manual_seed(seed)
    x = randn(gen, rows, D, bf16=bf16)
    gamma = randn(gen, D, scale=0.02, shift=1.0, bf16=bf16) if affine else None
    beta = randn(gen, D, scale=0.02, bf16=bf16) if affine and kind == "ln" else None
    dy = randn(gen, rows, D, bf16=bf16)
    rec = dict(kind=kind, rows=rows, D=D, eps=eps, act=act, affine=affine, bf16=bf16, x=x, dy=dy)
    if gamma is not None:
        rec["gamma"] = gamma
    if beta is not None:
        rec["beta"] = beta
    for tag, compute in (("f32", 0), ("f64", 1)):
        if kind == "ln":
            r = R.layernorm_act(x, gamma, beta, dy, eps, act, compute)
            keys = ("y", "dx", "dgamma", "dbeta")
            if compute == 1 and affine:
                rec["dgamma_f64x"], rec["dbeta_f64x"] = r["dgamma64"], r["dbeta64"]
        else:
            r = R.rmsnorm_act(x, gamma, dy, eps, act, compute)
            keys = ("y", "dx", "dweight")
            if compute == 1 and affine:
                rec["dweight_f64x"] = r["dweight64"]
        for k in keys:
            if r[k] is not None:
                rec[f"{k}_{tag}"] = r[k]
    return rec


def main():
    build_ref.build_reference()
    R.set_num_threads(1)
    cases = {}
    # LayerNorm (+act): the shapes of the benchmark configurations cut down to a few rows,
    # BERT's eps, an odd width, and a no-affine module.
    cases["ln_d512_none"] = norm_case("ln", 0, 16, 512, 1e-5, 0)
    cases["ln_d1024_gelu"] = norm_case("ln", 1, 8, 1024, 1e-5, 1)
    cases["ln_d7_silu_eps1e-12"] = norm_case("ln", 2, 5, 7, 1e-12, 2)
    cases["ln_d2048_gelu_noaffine"] = norm_case("ln", 3, 3, 2048, 1e-5, 1, affine=False)
    cases["ln_d768_gelu_bf16"] = norm_case("ln", 4, 6, 768, 1e-5, 1, bf16=True)
    cases["rms_d4096_none_bf16"] = norm_case("rms", 5, 4, 4096, 1e-6, 0, bf16=True)
    cases["rms_d768_silu"] = norm_case("rms", 6, 6, 768, 1e-6, 2)
    cases["rms_d33_gelu_noweight"] = norm_case("rms", 7, 4, 33, 1e-6, 1, affine=False)
    for name, rec in cases.items():
        np.savez(OUT / f"{name}.npz", **rec)

    gen = torch.Generator().manual_seed(10)
    x = np.concatenate([randn(gen, 900, scale=3.0), np.linspace(-30, 30, 124, dtype=np.float32)])
    dy = randn(gen, x.size)
    rec = dict(x=x, dy=dy)
    for act, nm in ((1, "gelu"), (2, "silu")):
        for tag, compute in (("f32", 0), ("f64", 1)):
            r = R.act(x, dy, act, compute)
            rec[f"{nm}_y_{tag}"], rec[f"{nm}_dx_{tag}"] = r["y"], r["dx"]
    np.savez(OUT / "act_gelu_silu.npz", **rec)

    gen = torch.Generator().manual_seed(11)
    inp = randn(gen, 8, 192)
    dy = randn(gen, 8, 96)
    rec = dict(input=inp, dy=dy)
    for tag, compute in (("f32", 0), ("f64", 1)):
        r = R.swiglu(inp, dy, compute)
        rec[f"swiglu_out_{tag}"], rec[f"swiglu_dinput_{tag}"] = r["out"], r["dinput"]
        m = R.mamba_gate(inp[:, :96].copy(), inp[:, 96:].copy(), dy, compute)
        rec[f"mamba_out_{tag}"], rec[f"mamba_dgate_{tag}"], rec[f"mamba_dup_{tag}"] = m["out"], m["dgate"], m["dup"]
    np.savez(OUT / "silu_gate.npz", **rec)

    # residual add + norm (classic.hpp:442-445 with LayerNorm, mamba.hpp:409-415 with RMSNorm)
    for name, kind, seed, rows, D, eps, bf16 in (("add_ln_d1024", "ln", 20, 6, 1024, 1e-5, False),
                                                 ("add_rms_d2048_bf16", "rms", 21, 5, 2048, 1e-6, True)):
        gen = torch.Generator().manual_seed(seed)
        a, b = randn(gen, rows, D, bf16=bf16), randn(gen, rows, D, bf16=bf16)
        gamma = randn(gen, D, scale=0.02, shift=1.0, bf16=bf16)
        beta = randn(gen, D, scale=0.02, bf16=bf16) if kind == "ln" else None
        dy, dsum = randn(gen, rows, D, bf16=bf16), randn(gen, rows, D, bf16=bf16)
        rec = dict(kind=kind, rows=rows, D=D, eps=eps, bf16=bf16, a=a, b=b, gamma=gamma, dy=dy, dsum=dsum)
        if beta is not None:
            rec["beta"] = beta
        for tag, compute in (("f32", 0), ("f64", 1)):
            r = R.add_norm(kind, a, b, gamma, beta, dy, dsum, eps, compute)
            for k in ("sum", "y", "da", "dgamma", "dbeta"):
                if r[k] is not None:
                    rec[f"{k}_{tag}"] = r[k]
        np.savez(OUT / f"{name}.npz", **rec)

    # BertEmbedding: word + position + type gathers and LayerNorm eps 1e-12 (bert.hpp:116-204)
    gen = torch.Generator().manual_seed(30)
    vocab, max_pos, tv, D, B, S = 50, 16, 2, 96, 3, 7
    word, pos, typ = randn(gen, vocab, D, scale=0.02), randn(gen, max_pos, D, scale=0.02), randn(gen, tv, D, scale=0.02)
    gamma, beta = randn(gen, D, scale=0.02, shift=1.0), randn(gen, D, scale=0.02)
    ids = torch.randint(0, vocab, (B, S), generator=gen).numpy().astype(np.int64)
    dy = randn(gen, B, S, D)
    rec = dict(word=word, pos=pos, type=typ, gamma=gamma, beta=beta, ids=ids, dy=dy)
    for tag, compute in (("f32", 0), ("f64", 1)):
        r = R.bert_embedding(word, pos, typ, gamma, beta, ids, dy, compute)
        for k, v in r.items():
            rec[f"{k}_{tag}"] = v
    np.savez(OUT / "bert_embedding.npz", **rec)
    # the same module fed ready-made embeddings (bert.hpp:164-171)
    inp = randn(gen, B, S, D, scale=0.5)
    rec = dict(input=inp, pos=pos, type=typ, gamma=gamma, beta=beta, dy=dy)
    for tag, compute in (("f32", 0), ("f64", 1)):
        r = R.bert_embedding_from_embeddings(inp, pos, typ, gamma, beta, dy, compute)
        for k, v in r.items():
            rec[f"{k}_{tag}"] = v
    np.savez(OUT / "bert_embedding_float_input.npz", **rec)

    # FC layer: torch::nn::Linear then apply(activation) (fc.hpp:31-49), bf16-representable operands
    gen = torch.Generator().manual_seed(50)
    M, N, K = 24, 40, 64
    fx, fw, fb = randn(gen, M, K, bf16=True), randn(gen, N, K, scale=0.1, bf16=True), randn(gen, N, scale=0.1, bf16=True)
    rec = dict(x=fx, weight=fw, bias=fb)
    for act_name, code in (("none", 0), ("gelu", 1), ("silu", 2)):
        for tag, compute in (("f32", 0), ("f64", 1)):
            r = R.fc_act(fx, fw, fb, code, compute)
            rec[f"{act_name}_y_{tag}"] = r["y"]
            rec[f"z_{tag}"] = r["z"]
    rec["nobias_gelu_y_f64"] = R.fc_act(fx, fw, None, 1, 1)["y"]
    np.savez(OUT / "fc_act.npz", **rec)

    gen = torch.Generator().manual_seed(12)
    table = randn(gen, 64, 40, scale=0.02)
    ids = torch.randint(0, 64, (3, 9), generator=gen).numpy().astype(np.int64)
    dout = randn(gen, 27, 40)
    r = R.token_embedding(table, ids, dout, 0)
    r64 = R.token_embedding(table, ids, dout, 1)
    np.savez(OUT / "embedding.npz", table=table, ids=ids, dout=dout, out=r["out"], dtable_f32=r["dtable"],
             dtable_f64=r64["dtable"])
    # Attention probabilities through the reference's ScaledDotProductKernel with key = value = identity
    # (kernel.hpp:20-94): key padding, additive masks of each accepted rank, causal; scale = 1/sqrt(S).
    gen = torch.Generator().manual_seed(40)
    B, H, T, S = 2, 3, 10, 24
    scores = randn(gen, B, H, T, S, scale=3.0)
    dattn = randn(gen, B, H, T, S)
    padding = np.zeros((B, S), np.uint8)
    padding[1, -7:] = 1
    rec = dict(scores=scores, dattn=dattn, padding=padding, mask2=randn(gen, T, S), mask3=randn(gen, B, T, S),
               mask4=randn(gen, B, H, T, S))
    rec["mask2"][2, :5] = -np.inf                     # a float mask may carry -inf itself
    cases = {"plain": (None, None, False), "causal": (None, None, True), "padding": ("padding", None, False),
             "mask2": (None, "mask2", False), "mask3_padding": ("padding", "mask3", False), "mask4_causal": (None, "mask4", True)}
    for name, (pk, mk, causal) in cases.items():
        for tag, compute in (("f32", 0), ("f64", 1)):
            r = R.attention_softmax(scores, rec[pk] if pk else None, rec[mk] if mk else None, causal, dattn, compute)
            rec[f"{name}_attn_{tag}"] = r["attn"]
            rec[f"{name}_dscores_{tag}"] = r["dscores"]
    np.savez(OUT / "attention_softmax.npz", **rec)
    # ... followed by the reference's multiplicative-noise dropout (dropout.hpp:32-51), p = 0.25, seeded; the stored
    # noise is the tensor the module drew
    drop = dict(scores=scores, dout=dattn, padding=padding, mask3=rec["mask3"], p=0.25, seed=1234)
    for name, (pk, mk, causal) in {"plain": (None, None, False), "mask3_padding_causal": ("padding", "mask3", True)}.items():
        for tag, compute in (("f32", 0), ("f64", 1)):
            r = R.attention_softmax_dropout(scores, 0.25, 1234, rec[pk] if pk else None, rec[mk] if mk else None, causal, dattn, compute)
            for k, v in r.items():
                drop[f"{name}_{k}_{tag}"] = v
    np.savez(OUT / "attention_softmax_dropout.npz", **drop)
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))


if __name__ == "__main__":
    main()
