"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: numpy front end of oracle_rowops.c.

Inputs are fp32 numpy arrays (bf16 cases pass bf16-representable fp32 values);
outputs are float64 arrays, which the tests round to the precision under test.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_int64, c_void_p

import numpy as np

from . import build_ref

ACT_NONE, ACT_GELU, ACT_SILU = 0, 1, 2
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_ref.C_LIB if build_ref.C_LIB.exists() else build_ref.build_c_oracle()
        _lib = ctypes.CDLL(str(path))
        _lib.orc_embedding.restype = c_int64
    return _lib


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else c_void_p(a.ctypes.data)


def layernorm_act(x, gamma, beta, dy, eps, act=ACT_NONE):
    x, gamma, beta, dy = _f32(x), _f32(gamma), _f32(beta), _f32(dy)
    rows, D = x.shape
    y = np.empty((rows, D)); mean = np.empty(rows); rstd = np.empty(rows)
    dx = np.empty((rows, D)) if dy is not None else None
    dg = np.empty(D) if dy is not None else None
    db = np.empty(D) if dy is not None else None
    lib().orc_layernorm_act(_p(x), _p(gamma), _p(beta), _p(dy), c_int64(rows), c_int64(D), c_double(eps), c_int(act),
                            _p(y), _p(mean), _p(rstd), _p(dx), _p(dg), _p(db))
    return dict(y=y, mean=mean, rstd=rstd, dx=dx, dgamma=dg, dbeta=db)


def rmsnorm_act(x, weight, dy, eps, act=ACT_NONE):
    x, weight, dy = _f32(x), _f32(weight), _f32(dy)
    rows, D = x.shape
    y = np.empty((rows, D)); rstd = np.empty(rows)
    dx = np.empty((rows, D)) if dy is not None else None
    dw = np.empty(D) if dy is not None else None
    lib().orc_rmsnorm_act(_p(x), _p(weight), _p(dy), c_int64(rows), c_int64(D), c_double(eps), c_int(act),
                          _p(y), _p(rstd), _p(dx), _p(dw))
    return dict(y=y, rstd=rstd, dx=dx, dweight=dw)


def act(x, dy, act_code):
    x, dy = _f32(x), _f32(dy)
    y = np.empty(x.shape); dx = np.empty(x.shape) if dy is not None else None
    lib().orc_act(_p(x), _p(dy), c_int64(x.size), c_int(act_code), _p(y), _p(dx))
    return dict(y=y, dx=dx)


def linear_act(x, weight, bias, act_code):
    """The FC layer of the reference (torch::nn::Linear then apply(activation), src/layer/details/fc.hpp:31-49):
    z = x @ weight.T + bias in fp64 on the given fp32 values, y = act(z) -> dict(z, y)."""
    z = np.asarray(x, np.float64) @ np.asarray(weight, np.float64).T
    if bias is not None:
        z = z + np.asarray(bias, np.float64)
    return dict(z=z, y=act64(z, act_code))


def act64(z, act_code):
    """GELU (exact erf) / SiLU / identity in fp64 on fp64 input (gelu.hpp:11-15, silu.hpp:12-16)."""
    from math import erf, sqrt
    z = np.asarray(z, np.float64)
    if act_code == ACT_GELU:
        return 0.5 * z * (1.0 + np.vectorize(erf)(z / sqrt(2.0)))
    if act_code == ACT_SILU:
        return z / (1.0 + np.exp(-z))
    return z.copy()


def silu_gate(a, b, dy):
    """a, b: 2-D fp32 arrays, possibly row-strided views with unit column stride."""
    assert a.dtype == np.float32 and b.dtype == np.float32
    assert a.strides[1] == 4 and b.strides[1] == 4
    rows, H = a.shape
    dy = _f32(dy)
    out = np.empty((rows, H))
    da = np.empty((rows, H)) if dy is not None else None
    db = np.empty((rows, H)) if dy is not None else None
    lib().orc_silu_gate(_p(a), c_int64(a.strides[0] // 4), _p(b), c_int64(b.strides[0] // 4), _p(dy), c_int64(H),
                        c_int64(rows), c_int64(H), _p(out), _p(da), _p(db))
    return dict(out=out, da=da, db=db)


def embedding(table, ids):
    """table: any 2-D array (rows copied byte for byte); -> (out, first bad position or -1)."""
    table = np.ascontiguousarray(table)
    ids = np.ascontiguousarray(ids, dtype=np.int64).reshape(-1)
    vocab, D = table.shape
    out = np.empty((ids.size, D), dtype=table.dtype)
    bad = lib().orc_embedding(_p(table), _p(ids), c_int64(ids.size), c_int64(vocab),
                              c_int64(D * table.dtype.itemsize), _p(out))
    return out, int(bad)


def embedding_bwd(dout, ids, vocab):
    dout = _f32(dout)
    ids = np.ascontiguousarray(ids, dtype=np.int64).reshape(-1)
    D = dout.shape[-1]
    dtable = np.empty((vocab, D))
    lib().orc_embedding_bwd(_p(dout), _p(ids), c_int64(ids.size), c_int64(vocab), c_int64(D), _p(dtable))
    return dtable


def rope_table(S, hd, theta=10000.0, positions=None):
    cs = np.empty((S, hd // 2, 2), dtype=np.float32)
    pos = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    lib().orc_rope_table(_p(pos), c_int64(S), c_int64(hd), c_double(theta), _p(cs))
    return cs


def rope_apply(x, cos_sin, inverse=False):
    x = _f32(x)
    B, S, H, hd = x.shape
    out = np.empty(x.shape)
    lib().orc_rope_apply(_p(x), _p(np.ascontiguousarray(cos_sin, dtype=np.float32)), c_int64(B), c_int64(S),
                         c_int64(H), c_int64(hd), c_int(int(inverse)), _p(out))
    return out


def add_norm(kind, a, b, gamma, beta, dy, dsum, eps, bf16=False):
    """Residual add in front of a norm: `output = residual + attention; norm(output)`
    (classic.hpp:442-445 LayerNorm, mamba.hpp:409-415 RMSNorm).  The sum is rounded to the
    tensor dtype before it is normalised, as the reference's sum tensor is.  da == db == dx."""
    s = (_f32(a).astype(np.float64) + _f32(b).astype(np.float64)).astype(np.float32)   # fp32 add of fp32/bf16 values
    if bf16:
        u = s.view(np.uint32).astype(np.uint64)
        s = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)
    r = layernorm_act(s, gamma, beta, dy, eps) if kind == "ln" else rmsnorm_act(s, gamma, dy, eps)
    out = dict(sum=s, y=r["y"], dgamma=r.get("dgamma", r.get("dweight")), dbeta=r.get("dbeta"))
    if dy is not None:
        out["dx"] = r["dx"] + (0.0 if dsum is None else _f32(dsum).astype(np.float64))
    return out


def bert_embedding(word, pos, type_table, gamma, beta, ids, dy=None, eps=1e-12, bf16=False):
    """BertEmbeddingImpl::forward (src/block/details/transformers/bert.hpp:155-194): word gather by
    id, position gather of arange(S), token-type gather of zeros (row 0), sum, LayerNorm(eps 1e-12).
    With dy: gradients of the three tables (type: row 0 only) and of gamma/beta.
    ids None: `word` is a ready-made [B, S, D] embeddings tensor (the module's other input branch,
    bert.hpp:164-171); dword is then not produced and dsum is the gradient of that input."""
    word = _f32(word)
    if ids is None:
        B, S, D = word.shape
        vocab = B * S
        word = word.reshape(B * S, D)
        ids = np.arange(B * S, dtype=np.int64).reshape(B, S)
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    B, S = ids.shape
    vocab, D = word.shape
    # the three rows are added one after the other in fp32, as tensor adds are
    s = word[ids.reshape(-1)].astype(np.float32)
    if pos is not None:
        s = (s + np.tile(_f32(pos)[:S], (B, 1))).astype(np.float32)
    if type_table is not None:
        s = (s + _f32(type_table)[0]).astype(np.float32)
    if bf16:
        s = _round_bf16(s)
    r = layernorm_act(s, gamma, beta, None if dy is None else _f32(dy).reshape(B * S, D), eps)
    out = dict(sum=s, y=r["y"].reshape(B, S, D), dgamma=r["dgamma"], dbeta=r["dbeta"])
    if dy is not None:
        dx = r["dx"]
        if bf16:      # the gradient of the sum is itself a bf16 tensor before it is scattered / reduced
            dx = _round_bf16(dx.astype(np.float32)).astype(np.float64)
        out["dsum"] = dx
        out["dword"] = _scatter_rows(dx, ids.reshape(-1), vocab)
        out["dpos"] = dx.reshape(B, S, D).sum(axis=0)
        out["dtype0"] = dx.sum(axis=0)
    return out


def _mask_strides(attn_mask, B, H, T, S):
    if attn_mask is None:
        return 0, 0
    if attn_mask.ndim == 2:
        return 0, 0
    if attn_mask.ndim == 3 and attn_mask.shape[0] == B:
        return T * S, 0
    return H * T * S, T * S


def attention_softmax(scores, scale, key_padding=None, attn_mask=None, causal=False, dattn=None, noise=None):
    """scores [B,H,T,S] fp32 -> dict(attn, dscores) in fp64 (kernel.hpp:33-93).  With `noise` (the dropout's
    multiplicative noise, kernel.hpp:94 / dropout.hpp:41-43) also `dropped` = attn * noise, and dattn is the
    gradient of `dropped`."""
    scores, attn_mask, dattn, noise = _f32(scores), _f32(attn_mask), _f32(dattn), _f32(noise)
    B, H, T, S = scores.shape
    kp = None if key_padding is None else np.ascontiguousarray(key_padding, dtype=np.uint8)
    sb, sh = _mask_strides(attn_mask, B, H, T, S)
    attn = np.empty(scores.shape)
    ds = np.empty(scores.shape) if dattn is not None else None
    dropped = np.empty(scores.shape) if noise is not None else None
    with np.errstate(invalid="ignore"):
        lib().orc_attention_softmax_noise(_p(scores), _p(kp), _p(attn_mask), c_int64(sb), c_int64(sh), _p(dattn), _p(noise), c_int64(B),
                                          c_int64(H), c_int64(T), c_int64(S), c_double(scale), c_int(int(causal)), _p(attn), _p(dropped),
                                          _p(ds))
    return dict(attn=attn, dscores=ds, dropped=dropped)


def _round_bf16(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def _scatter_rows(dx, ids, vocab):
    out = np.zeros((vocab, dx.shape[1]))
    np.add.at(out, ids, dx)
    return out
