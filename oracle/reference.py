"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: numpy front end of oracle/_ref/libnott_ref.so,
the reference's own modules (compiled from its headers) running on libtorch CPU.

compute: 0 = fp32, 1 = fp64, 2 = native bf16 (see ref_harness.cpp).
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_int64, c_void_p

import numpy as np

from . import build_ref

_lib = None


def available() -> bool:
    return build_ref.REF_LIB.exists()


def lib():
    global _lib
    if _lib is None:
        import torch  # noqa: F401  (loads libtorch before the harness resolves it)

        if not build_ref.REF_LIB.exists():
            raise RuntimeError("oracle/_ref/libnott_ref.so is not built (needs the reference checkout)")
        _lib = ctypes.CDLL(str(build_ref.REF_LIB))
        _lib.ref_last_error.restype = ctypes.c_char_p
        _lib.ref_time_norm_act.restype = c_double
    return _lib


def _chk(rc):
    if rc != 0:
        raise RuntimeError("reference harness: " + lib().ref_last_error().decode())


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else c_void_p(a.ctypes.data)


def num_threads() -> int:
    return int(lib().ref_get_num_threads())


def set_num_threads(n: int) -> None:
    lib().ref_set_num_threads(c_int(n))


def layernorm_act(x, gamma, beta, dy, eps, act=0, compute=0):
    x, gamma, beta, dy = _f32(x), _f32(gamma), _f32(beta), _f32(dy)
    rows, D = x.shape
    y = np.empty((rows, D), np.float32)
    bwd = dy is not None
    dx = np.empty((rows, D), np.float32) if bwd else None
    aff = bwd and gamma is not None
    dg = np.empty(D, np.float32) if aff else None
    db = np.empty(D, np.float32) if aff else None
    dg64 = np.empty(D, np.float64) if aff else None
    db64 = np.empty(D, np.float64) if aff else None
    _chk(lib().ref_layernorm_act(_p(x), _p(gamma), _p(beta), _p(dy), c_int64(rows), c_int64(D), c_double(eps),
                                 c_int(act), c_int(compute), _p(y), _p(dx), _p(dg), _p(db), _p(dg64), _p(db64)))
    return dict(y=y, dx=dx, dgamma=dg, dbeta=db, dgamma64=dg64, dbeta64=db64)


def rmsnorm_act(x, weight, dy, eps, act=0, compute=0):
    x, weight, dy = _f32(x), _f32(weight), _f32(dy)
    rows, D = x.shape
    y = np.empty((rows, D), np.float32)
    bwd = dy is not None
    dx = np.empty((rows, D), np.float32) if bwd else None
    dw = np.empty(D, np.float32) if bwd and weight is not None else None
    dw64 = np.empty(D, np.float64) if bwd and weight is not None else None
    _chk(lib().ref_rmsnorm_act(_p(x), _p(weight), _p(dy), c_int64(rows), c_int64(D), c_double(eps), c_int(act),
                               c_int(compute), _p(y), _p(dx), _p(dw), _p(dw64)))
    return dict(y=y, dx=dx, dweight=dw, dweight64=dw64)


def add_norm(kind, a, b, gamma, beta, dy, dsum, eps, compute=0):
    a, b, gamma, beta, dy, dsum = map(_f32, (a, b, gamma, beta, dy, dsum))
    rows, D = a.shape
    s = np.empty((rows, D), np.float32); y = np.empty((rows, D), np.float32)
    bwd = dy is not None
    da = np.empty((rows, D), np.float32) if bwd else None
    dg = np.empty(D, np.float32) if bwd else None
    db = np.empty(D, np.float32) if bwd and kind == "ln" else None
    _chk(lib().ref_add_norm(c_int(1 if kind == "rms" else 0), _p(a), _p(b), _p(gamma), _p(beta), _p(dy), _p(dsum),
                            c_int64(rows), c_int64(D), c_double(eps), c_int(compute), _p(s), _p(y), _p(da), _p(dg), _p(db)))
    return dict(sum=s, y=y, da=da, dgamma=dg, dbeta=db)


def bert_embedding(word, pos, type_table, gamma, beta, ids, dy=None, compute=0):
    word, pos, type_table, gamma, beta, dy = map(_f32, (word, pos, type_table, gamma, beta, dy))
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    B, S = ids.shape
    vocab, D = word.shape
    max_pos = pos.shape[0] if pos is not None else 0
    tv = type_table.shape[0] if type_table is not None else 0
    y = np.empty((B, S, D), np.float32)
    bwd = dy is not None
    dword = np.empty((vocab, D), np.float32) if bwd else None
    dpos = np.empty((max_pos, D), np.float32) if bwd and pos is not None else None
    dtype = np.empty((tv, D), np.float32) if bwd and type_table is not None else None
    dg = np.empty(D, np.float32) if bwd else None
    db = np.empty(D, np.float32) if bwd else None
    _chk(lib().ref_bert_embedding(_p(word), _p(pos), _p(type_table), _p(gamma), _p(beta), _p(ids), _p(dy), c_int64(B), c_int64(S),
                                  c_int64(vocab), c_int64(max_pos), c_int64(tv), c_int64(D), c_int(compute),
                                  _p(y), _p(dword), _p(dpos), _p(dtype), _p(dg), _p(db)))
    return dict(y=y, dword=dword, dpos=dpos, dtype=dtype, dgamma=dg, dbeta=db)


def fc_act(x, weight, bias, act_code, compute=0):
    """torch::nn::Linear then apply(activation), the reference's FC layer (fc.hpp:31-49) -> dict(z, y)."""
    x, weight, bias = _f32(x), _f32(weight), _f32(bias)
    M, K = x.shape
    N = weight.shape[0]
    z = np.empty((M, N), np.float32); y = np.empty((M, N), np.float32)
    _chk(lib().ref_fc_act(_p(x), _p(weight), _p(bias), c_int64(M), c_int64(N), c_int64(K), c_int(act_code), c_int(compute), _p(z), _p(y)))
    return dict(z=z, y=y)


def bert_embedding_from_embeddings(inp, pos, type_table, gamma, beta, dy=None, compute=0):
    """BertEmbedding fed ready-made [B, S, D] embeddings (bert.hpp:164-171) instead of token ids."""
    inp, pos, type_table, gamma, beta, dy = map(_f32, (inp, pos, type_table, gamma, beta, dy))
    B, S, D = inp.shape
    max_pos = pos.shape[0] if pos is not None else 0
    tv = type_table.shape[0] if type_table is not None else 0
    y = np.empty((B, S, D), np.float32)
    bwd = dy is not None
    dinp = np.empty((B, S, D), np.float32) if bwd else None
    dpos = np.empty((max_pos, D), np.float32) if bwd and pos is not None else None
    dtype = np.empty((tv, D), np.float32) if bwd and type_table is not None else None
    dg = np.empty(D, np.float32) if bwd else None
    db = np.empty(D, np.float32) if bwd else None
    _chk(lib().ref_bert_embedding_from_embeddings(_p(inp), _p(pos), _p(type_table), _p(gamma), _p(beta), _p(dy), c_int64(B), c_int64(S),
                                                  c_int64(max_pos), c_int64(tv), c_int64(D), c_int(compute),
                                                  _p(y), _p(dinp), _p(dpos), _p(dtype), _p(dg), _p(db)))
    return dict(y=y, dinput=dinp, dpos=dpos, dtype=dtype, dgamma=dg, dbeta=db)


def act(x, dy, act_code, compute=0):
    x, dy = _f32(x), _f32(dy)
    y = np.empty(x.shape, np.float32)
    dx = np.empty(x.shape, np.float32) if dy is not None else None
    _chk(lib().ref_act(_p(x), _p(dy), c_int64(x.size), c_int(act_code), c_int(compute), _p(y), _p(dx)))
    return dict(y=y, dx=dx)


def swiglu(inp, dy, compute=0):
    inp, dy = _f32(inp), _f32(dy)
    rows, H2 = inp.shape
    H = H2 // 2
    out = np.empty((rows, H), np.float32)
    dinp = np.empty((rows, H2), np.float32) if dy is not None else None
    _chk(lib().ref_swiglu(_p(inp), _p(dy), c_int64(rows), c_int64(H), c_int(compute), _p(out), _p(dinp)))
    return dict(out=out, dinput=dinp)


def mamba_gate(gate, up, dy, compute=0):
    gate, up, dy = _f32(gate), _f32(up), _f32(dy)
    rows, H = gate.shape
    out = np.empty((rows, H), np.float32)
    dg = np.empty((rows, H), np.float32) if dy is not None else None
    du = np.empty((rows, H), np.float32) if dy is not None else None
    _chk(lib().ref_mamba_gate(_p(gate), _p(up), _p(dy), c_int64(rows), c_int64(H), c_int(compute), _p(out), _p(dg), _p(du)))
    return dict(out=out, dgate=dg, dup=du)


def token_embedding(table, ids, dout=None, compute=0):
    table, dout = _f32(table), _f32(dout)
    ids = np.ascontiguousarray(ids, dtype=np.int64).reshape(-1)
    vocab, D = table.shape
    out = np.empty((ids.size, D), np.float32)
    dtable = np.empty((vocab, D), np.float32) if dout is not None else None
    _chk(lib().ref_token_embedding(_p(table), _p(ids), _p(dout), c_int64(ids.size), c_int64(vocab), c_int64(D),
                                   c_int(compute), _p(out), _p(dtable)))
    return dict(out=out, dtable=dtable)


def attention_softmax(scores, key_padding=None, attn_mask=None, causal=False, dattn=None, compute=0):
    """The reference's ScaledDotProductKernel with key = value = identity: scale is 1/sqrt(S)."""
    scores, attn_mask, dattn = _f32(scores), _f32(attn_mask), _f32(dattn)
    B, H, T, S = scores.shape
    kp = None if key_padding is None else np.ascontiguousarray(key_padding, dtype=np.uint8)
    attn = np.empty(scores.shape, dtype=np.float32)
    ds = np.empty(scores.shape, dtype=np.float32) if dattn is not None else None
    dims = 0 if attn_mask is None else attn_mask.ndim
    _chk(lib().ref_attention_softmax(_p(scores), _p(kp), _p(attn_mask), c_int(dims), _p(dattn), c_int64(B), c_int64(H),
                                     c_int64(T), c_int64(S), c_int(int(causal)), c_int(compute), _p(attn), _p(ds)))
    return dict(attn=attn, dscores=ds)


def attention_softmax_dropout(scores, p, seed, key_padding=None, attn_mask=None, causal=False, dout=None, compute=0):
    """ScaledDotProductKernel's probabilities (key = value = identity) followed by the reference's HardDropout
    (input * N(1, sqrt(p/(1-p)))) seeded with `seed`; also returns the noise tensor the module drew."""
    scores, attn_mask, dout = _f32(scores), _f32(attn_mask), _f32(dout)
    B, H, T, S = scores.shape
    kp = None if key_padding is None else np.ascontiguousarray(key_padding, dtype=np.uint8)
    attn = np.empty(scores.shape, dtype=np.float32); noise = np.empty(scores.shape, dtype=np.float32)
    out = np.empty(scores.shape, dtype=np.float32)
    ds = np.empty(scores.shape, dtype=np.float32) if dout is not None else None
    dims = 0 if attn_mask is None else attn_mask.ndim
    _chk(lib().ref_attention_softmax_dropout(_p(scores), _p(kp), _p(attn_mask), c_int(dims), _p(dout), c_int64(B), c_int64(H),
                                             c_int64(T), c_int64(S), c_int(int(causal)), c_double(p), c_int64(seed), c_int(compute),
                                             _p(attn), _p(noise), _p(out), _p(ds)))
    return dict(attn=attn, noise=noise, out=out, dscores=ds)


def time_norm_act(kind, rows, D, eps, act, compute=0, iters=10, warmup=2) -> float:
    """Seconds per forward+backward of the reference modules, timed inside the harness."""
    t = lib().ref_time_norm_act(c_int(1 if kind == "rms" else 0), c_int64(rows), c_int64(D), c_double(eps),
                                c_int(act), c_int(compute), c_int(iters), c_int(warmup))
    if t < 0:
        raise RuntimeError("reference harness: " + lib().ref_last_error().decode())
    return float(t)


# ---- the reference's RegisteredLayer / ForwardBinding driving the drop-in modules (libnott_binding.so)
_bind = None


def binding_available() -> bool:
    return build_ref.BINDING_LIB.exists()


def binding_lib():
    global _bind
    if _bind is None:
        import torch  # noqa: F401

        if not build_ref.BINDING_LIB.exists():
            raise RuntimeError("oracle/_ref/libnott_binding.so is not built (needs the reference checkout)")
        _bind = ctypes.CDLL(str(build_ref.BINDING_LIB))
        _bind.refbind_last_error.restype = ctypes.c_char_p
    return _bind


BIND_MODULE, BIND_COPY, BIND_INLINE_COPY_MOVE, BIND_REFERENCE_F32, BIND_REFERENCE_F64 = range(5)


def binding_layernorm_gelu(which, x, dy, gamma, beta, eps=1e-5, bf16=False):
    """`layer.forward(x)` then `apply(layer.activation, .)` through a RegisteredLayer, plus backward.
    which: BIND_MODULE / BIND_COPY / BIND_INLINE_COPY_MOVE run Nott::B200::LayerNorm (GeLU fused) on CUDA,
    BIND_REFERENCE_F32 / _F64 the reference pair torch::nn::LayerNorm + apply(GeLU) on CPU.  x, dy: [B, S, D]."""
    x, dy, gamma, beta = _f32(x), _f32(dy), _f32(gamma), _f32(beta)
    B, S, D = x.shape
    y = np.empty((B, S, D), np.float32); dx = np.empty((B, S, D), np.float32)
    dg = np.empty(D, np.float32); db = np.empty(D, np.float32)
    rc = binding_lib().refbind_layernorm_gelu(c_int(which), _p(x), _p(dy), _p(gamma), _p(beta), c_int64(B), c_int64(S), c_int64(D),
                                              c_double(eps), c_int(int(bf16)), _p(y), _p(dx), _p(dg), _p(db))
    if rc != 0:
        raise RuntimeError("binding harness: " + binding_lib().refbind_last_error().decode())
    return dict(y=y, dx=dx, dgamma=dg, dbeta=db)
