"""The plain-C oracle (oracle/oracle_rowops.c) against the committed outputs of the
reference's own modules (tests/golden/*.npz, made by tests/golden/make_golden.py)."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import cpu_oracle as O
from tests import tol

NORM_CASES = ["ln_d512_none", "ln_d1024_gelu", "ln_d7_silu_eps1e-12", "ln_d2048_gelu_noaffine",
              "ln_d768_gelu_bf16", "rms_d4096_none_bf16", "rms_d768_silu", "rms_d33_gelu_noweight"]


def load(golden_dir, name):
    z = np.load(golden_dir / f"{name}.npz")
    return {k: z[k] for k in z.files}


@pytest.mark.parametrize("name", NORM_CASES)
def test_norm_oracle_matches_reference(golden_dir, name):
    g = load(golden_dir, name)
    eps, act = float(g["eps"]), int(g["act"])
    if str(g["kind"]) == "ln":
        o = O.layernorm_act(g["x"], g.get("gamma"), g.get("beta"), g["dy"], eps, act)
        sums = ("dgamma", "dbeta") if "gamma" in g else ()
    else:
        o = O.rmsnorm_act(g["x"], g.get("gamma"), g["dy"], eps, act)
        sums = ("dweight",) if "gamma" in g else ()
    for k in ("y", "dx"):
        tol.fp32_close(o[k], g[f"{k}_f32"])
        # the fp64 run of the reference modules is the tighter pin
        np.testing.assert_allclose(o[k], g[f"{k}_f64"], rtol=2e-6, atol=2e-7)
    for k in sums:
        tol.long_sum_close(o[k], g[f"{k}_f64x"], int(g["rows"]), ref32=g[f"{k}_f32"])
        np.testing.assert_allclose(o[k], g[f"{k}_f64x"], rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("name,code", [("gelu", O.ACT_GELU), ("silu", O.ACT_SILU)])
def test_activation_oracle_matches_reference(golden_dir, name, code):
    g = load(golden_dir, "act_gelu_silu")
    o = O.act(g["x"], g["dy"], code)
    tol.fp32_close(o["y"], g[f"{name}_y_f32"])
    tol.fp32_close(o["dx"], g[f"{name}_dx_f32"])
    np.testing.assert_allclose(o["y"], g[f"{name}_y_f64"], rtol=2e-6, atol=2e-7)
    np.testing.assert_allclose(o["dx"], g[f"{name}_dx_f64"], rtol=2e-6, atol=2e-7)


def test_silu_gate_oracle_matches_swiglu_and_mamba(golden_dir):
    g = load(golden_dir, "silu_gate")
    inp = g["input"]
    H = inp.shape[1] // 2
    o = O.silu_gate(inp[:, :H], inp[:, H:], g["dy"])            # row-strided halves, as SwiGLU sees them
    tol.fp32_close(o["out"], g["swiglu_out_f32"])
    tol.fp32_close(o["da"], g["swiglu_dinput_f32"][:, :H])
    tol.fp32_close(o["db"], g["swiglu_dinput_f32"][:, H:])
    np.testing.assert_allclose(o["out"], g["swiglu_out_f64"], rtol=2e-6, atol=2e-7)
    o2 = O.silu_gate(np.ascontiguousarray(inp[:, :H]), np.ascontiguousarray(inp[:, H:]), g["dy"])
    tol.fp32_close(o2["out"], g["mamba_out_f32"])
    tol.fp32_close(o2["da"], g["mamba_dgate_f32"])
    tol.fp32_close(o2["db"], g["mamba_dup_f32"])


def test_embedding_oracle_is_bit_exact(golden_dir):
    g = load(golden_dir, "embedding")
    out, bad = O.embedding(g["table"], g["ids"])
    assert bad == -1
    assert out.tobytes() == g["out"].tobytes()
    dt = O.embedding_bwd(g["dout"], g["ids"], g["table"].shape[0])
    tol.fp32_close(dt, g["dtable_f32"])
    np.testing.assert_allclose(dt, g["dtable_f64"], rtol=2e-6, atol=2e-7)


def test_embedding_oracle_flags_bad_ids():
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    out, bad = O.embedding(table, np.array([1, 7, -1, 3]))
    assert bad == 1
    assert (out[1] == 0).all() and (out[2] == 0).all()
    assert (out[0] == table[1]).all() and (out[3] == table[3]).all()


def test_rope_oracle_properties():
    # no reference implementation exists: check the definition's own invariants
    rng = np.random.default_rng(0)
    S, hd = 9, 16
    cs = O.rope_table(S, hd, 10000.0)
    assert cs.shape == (S, hd // 2, 2)
    assert np.allclose(cs[0, :, 0], 1.0) and np.allclose(cs[0, :, 1], 0.0)          # position 0: identity
    np.testing.assert_allclose(cs[..., 0] ** 2 + cs[..., 1] ** 2, 1.0, atol=1e-6)
    np.testing.assert_allclose(cs[3, 0], [np.cos(3.0), np.sin(3.0)], rtol=1e-6)     # i = 0: angle = pos
    x = rng.standard_normal((2, S, 3, hd)).astype(np.float32)
    y = O.rope_apply(x, cs)
    np.testing.assert_allclose((y ** 2).sum(-1), (x.astype(np.float64) ** 2).sum(-1), rtol=1e-6)   # a rotation
    back = O.rope_apply(y.astype(np.float32), cs, inverse=True)
    np.testing.assert_allclose(back, x, atol=1e-6)
    pos = np.array([5, 0, 2], dtype=np.int32)
    cs2 = O.rope_table(3, hd, 10000.0, positions=pos)
    assert np.array_equal(cs2[0], O.rope_table(6, hd)[5]) and np.array_equal(cs2[2], cs[2])


@pytest.mark.parametrize("name", ["add_ln_d1024", "add_rms_d2048_bf16"])
def test_residual_add_norm_oracle_matches_reference(golden_dir, name):
    g = load(golden_dir, name)
    kind, bf16 = str(g["kind"]), bool(g["bf16"])
    o = O.add_norm(kind, g["a"], g["b"], g["gamma"], g.get("beta"), g["dy"], g["dsum"], float(g["eps"]), bf16=False)
    # the fp32 run of the reference keeps the sum in fp32, so the un-rounded oracle sum is the one to compare
    assert np.array_equal(o["sum"], g["sum_f32"])
    tol.fp32_close(o["y"], g["y_f32"])
    tol.fp32_close(o["dx"], g["da_f32"])
    np.testing.assert_allclose(o["dx"], g["da_f64"], rtol=2e-6, atol=2e-6)
    tol.long_sum_close(o["dgamma"], g["dgamma_f64"], int(g["rows"]), ref32=g["dgamma_f32"])
    if kind == "ln":
        tol.long_sum_close(o["dbeta"], g["dbeta_f64"], int(g["rows"]), ref32=g["dbeta_f32"])
    if bf16:   # bf16 tensors: the reference's own sum tensor is a bf16 tensor, i.e. the rounded sum
        ob = O.add_norm(kind, g["a"], g["b"], g["gamma"], g.get("beta"), g["dy"], g["dsum"], float(g["eps"]), bf16=True)
        assert np.array_equal(tol.to_bf16_bits(g["sum_f32"]), tol.to_bf16_bits(ob["sum"]))


def test_bert_embedding_oracle_matches_reference_module(golden_dir):
    g = load(golden_dir, "bert_embedding")
    o = O.bert_embedding(g["word"], g["pos"], g["type"], g["gamma"], g["beta"], g["ids"], g["dy"])
    # eps = 1e-12 and table values ~0.02: rstd ~ 35, so the outputs are O(1) and the usual tolerance applies
    tol.fp32_close(o["y"], g["y_f32"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(o["y"], g["y_f64"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(o["dword"], g["dword_f64"], rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(o["dpos"], g["dpos_f64"][:7], rtol=1e-5, atol=1e-4)
    assert not g["dpos_f64"][7:].any()                       # positions beyond S get no gradient
    np.testing.assert_allclose(o["dtype0"], g["dtype_f64"][0], rtol=1e-5, atol=1e-4)
    assert not g["dtype_f64"][1].any()                       # token types are always 0 (bert.hpp:184)
    tol.long_sum_close(o["dgamma"], g["dgamma_f64"], 21, ref32=g["dgamma_f32"])
    tol.long_sum_close(o["dbeta"], g["dbeta_f64"], 21, ref32=g["dbeta_f32"])


def test_bert_embedding_oracle_with_ready_made_embeddings(golden_dir):
    """The module's other input branch (bert.hpp:164-171): a float [B, S, D] input is the embeddings themselves."""
    g = load(golden_dir, "bert_embedding_float_input")
    B, S, D = g["input"].shape
    o = O.bert_embedding(g["input"], g["pos"], g["type"], g["gamma"], g["beta"], None, g["dy"])
    tol.fp32_close(o["y"], g["y_f32"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(o["y"], g["y_f64"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(o["dsum"].reshape(B, S, D), g["dinput_f64"], rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(o["dpos"], g["dpos_f64"][:S], rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(o["dtype0"], g["dtype_f64"][0], rtol=1e-5, atol=1e-4)
    tol.long_sum_close(o["dgamma"], g["dgamma_f64"], B * S, ref32=g["dgamma_f32"])
    tol.long_sum_close(o["dbeta"], g["dbeta_f64"], B * S, ref32=g["dbeta_f32"])


ATTN_CASES = {"plain": (None, None, False), "causal": (None, None, True), "padding": ("padding", None, False),
              "mask2": (None, "mask2", False), "mask3_padding": ("padding", "mask3", False), "mask4_causal": (None, "mask4", True)}


@pytest.mark.parametrize("name", sorted(ATTN_CASES))
def test_attention_softmax_oracle_matches_reference_kernel(golden_dir, name):
    """Golden = the reference's ScaledDotProductKernel run with key = value = identity, so that its
    output is the attention matrix of the given scores (scale 1/sqrt(S))."""
    g = load(golden_dir, "attention_softmax")
    pk, mk, causal = ATTN_CASES[name]
    S = g["scores"].shape[-1]
    o = O.attention_softmax(g["scores"], 1.0 / np.sqrt(S), g[pk] if pk else None, g[mk] if mk else None, causal, g["dattn"])
    # the module ran in fp64 and its outputs were stored as fp32: agreement to fp32 rounding
    np.testing.assert_allclose(o["attn"], g[f"{name}_attn_f64"], rtol=1.2e-7, atol=1e-12)
    np.testing.assert_allclose(o["dscores"], g[f"{name}_dscores_f64"], rtol=1.2e-7, atol=1e-10)
    tol.fp32_close(o["attn"], g[f"{name}_attn_f32"])
    tol.fp32_close(o["dscores"], g[f"{name}_dscores_f32"])
    assert np.allclose(o["attn"].sum(-1), 1.0)
    if causal:
        assert not np.triu(o["attn"], 1).any()          # nothing attends to a later column


def test_attention_softmax_oracle_fully_masked_row_is_nan():
    scores = np.zeros((1, 1, 2, 4), np.float32)
    padding = np.ones((1, 4), np.uint8)
    o = O.attention_softmax(scores, 0.5, padding)
    assert np.isnan(o["attn"]).all()                     # torch::softmax of a row of -inf


@pytest.mark.parametrize("name", ["plain", "mask3_padding_causal"])
def test_attention_dropout_oracle_matches_reference_modules(golden_dir, name):
    """Golden = ScaledDotProductKernel's probabilities followed by the reference's HardDropout module
    (dropout.hpp:32-51), with the noise that module drew from the seeded generator."""
    g = load(golden_dir, "attention_softmax_dropout")
    use = name != "plain"
    S = g["scores"].shape[-1]
    for tag in ("f32", "f64"):
        noise = g[f"{name}_noise_{tag}"]
        o = O.attention_softmax(g["scores"], 1.0 / np.sqrt(S), g["padding"] if use else None, g["mask3"] if use else None, use,
                                g["dout"], noise=noise)
        tol.fp32_close(o["attn"], g[f"{name}_attn_{tag}"])
        tol.fp32_close(o["dropped"], g[f"{name}_out_{tag}"], rtol=2e-5, atol=2e-6)
        tol.fp32_close(o["dscores"], g[f"{name}_dscores_{tag}"], rtol=2e-5, atol=2e-6)
    # the module's noise has the moments it should: mean 1, std sqrt(p/(1-p))
    p = float(g["p"])
    assert abs(g["plain_noise_f32"].mean() - 1.0) < 0.05 and abs(g["plain_noise_f32"].std() - np.sqrt(p / (1 - p))) < 0.05


def test_fc_layer_oracle_matches_reference(golden_dir):
    """Golden = torch::nn::Linear followed by apply(activation), the reference's FC layer (fc.hpp:31-49)."""
    g = load(golden_dir, "fc_act")
    for name, code in (("none", O.ACT_NONE), ("gelu", O.ACT_GELU), ("silu", O.ACT_SILU)):
        o = O.linear_act(g["x"], g["weight"], g["bias"], code)
        np.testing.assert_allclose(o["y"], g[f"{name}_y_f64"], rtol=2e-7, atol=1e-7)      # fp64 module output stored as fp32
        tol.fp32_close(o["y"], g[f"{name}_y_f32"], rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(o["z"], g["z_f64"], rtol=2e-7, atol=1e-7)
    np.testing.assert_allclose(O.linear_act(g["x"], g["weight"], None, O.ACT_GELU)["y"], g["nobias_gelu_y_f64"], rtol=2e-7, atol=1e-7)
