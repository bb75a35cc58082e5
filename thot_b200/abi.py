"""ctypes binding of libnott_b200.so (the C ABI in include/nott_b200.h).

This is the thinnest possible host: it passes raw device pointers of torch
tensors to the extern "C" entry points on torch's current stream.  torch is
used only for device memory and streams.  If the library is missing or a call
fails, it raises; there is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_int, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

import torch

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU, ACT_SILU = 0, 1, 2
I32, I64 = 0, 1
WS_NORM_BWD, WS_EMBEDDING_BWD, WS_ROPE_TABLE, WS_BERT_EMBEDDING_BWD, WS_LINEAR = 0, 1, 2, 3, 4
EXCHANGE_NCCL, EXCHANGE_PEER = 0, 1
NORM_LAYER, NORM_RMS = 0, 1
COMM_ID_BYTES = 128
ERR_COMM, ERR_COMM_TIMEOUT = -7, -8

LIB_PATH = Path(__file__).resolve().parent / "libnott_b200.so"

_SIGNATURES = {
    "nb2_abi_version": (c_int, []),
    "nb2_last_error_string": (c_char_p, []),
    "nb2_sm_count": (c_int, []),
    "nb2_reserve_sms": (c_int, [c_int]),
    "nb2_device_status": (c_int, [POINTER(ctypes.c_uint), c_int]),
    "nb2_embedding_index": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "nb2_embedding_bwd_indexed": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "nb2_attention_softmax_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                          c_double, c_int, c_int, c_void_p]),
    "nb2_attention_softmax_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_double, c_int, c_void_p]),
    "nb2_attention_softmax_dropout_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                                  c_int64, c_int64, c_int64, c_int64, c_double, c_int, c_int, c_void_p]),
    "nb2_attention_softmax_dropout_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_double, c_int, c_void_p]),
    "nb2_linear_bias_act_fwd": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "nb2_linear_available": (c_int, []),
    "nb2_selftest_bounded_wait": (c_int, [c_int64, c_void_p, c_void_p]),
    "nb2_attention_softmax_order": (c_int, [c_int]),
    "nb2_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int]),
    "nb2_layernorm_fwd": (c_int, [c_void_p] * 6 + [c_int64, c_int64, c_double, c_int, c_int, c_void_p]),
    "nb2_layernorm_bwd": (c_int, [c_void_p] * 8 + [POINTER(c_int64), c_int64, c_int64, c_int, c_int, c_void_p]),
    "nb2_layernorm_bwd_static": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int, c_int, c_void_p]),
    "nb2_rmsnorm_fwd": (c_int, [c_void_p] * 4 + [c_int64, c_int64, c_double, c_int, c_int, c_void_p]),
    "nb2_rmsnorm_bwd": (c_int, [c_void_p] * 6 + [POINTER(c_int64), c_int64, c_int64, c_int, c_int, c_void_p]),
    "nb2_add_layernorm_fwd": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_double, c_int, c_void_p]),
    "nb2_add_layernorm_bwd": (c_int, [c_void_p] * 8 + [POINTER(c_int64), c_int64, c_int64, c_int, c_void_p]),
    "nb2_add_rmsnorm_fwd": (c_int, [c_void_p] * 6 + [c_int64, c_int64, c_double, c_int, c_void_p]),
    "nb2_add_rmsnorm_bwd": (c_int, [c_void_p] * 7 + [POINTER(c_int64), c_int64, c_int64, c_int, c_void_p]),
    "nb2_colreduce_partials": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "nb2_act_fwd": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "nb2_act_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "nb2_silu_gate_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nb2_silu_gate_bwd": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                  c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nb2_embedding_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nb2_embedding_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                                  c_void_p, c_size_t, c_void_p]),
    "nb2_bert_embedding_ln_fwd": (c_int, [c_void_p] * 10 + [c_int64, c_int64, c_int64, c_int64, c_double, c_int, c_int, c_void_p, c_void_p]),
    "nb2_bert_embedding_ln_bwd": (c_int, [c_void_p] * 9 + [c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                          c_void_p, c_size_t, c_void_p]),
    "nb2_rope_table": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_double, c_void_p]),
    "nb2_rope_apply": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "nb2_host_ctx_create": (c_int, [POINTER(c_void_p), c_int64, c_int64, c_int, c_int64]),
    "nb2_host_ctx_destroy": (c_int, [c_void_p]),
    "nb2_layernorm_act_step_host": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_double, c_int, c_int]),
    "nb2_rmsnorm_act_step_host": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_double, c_int, c_int]),
    "nb2_comm_unique_id": (c_int, [c_void_p]),
    "nb2_comm_create": (c_int, [POINTER(c_void_p), c_void_p, c_int, c_int, c_int, c_int64]),
    "nb2_comm_destroy": (c_int, [c_void_p]),
    "nb2_comm_info": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "nb2_grad_exchange_begin": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "nb2_grad_exchange_end": (c_int, [c_void_p, c_void_p]),
    "nb2_comm_wait": (c_int, [c_void_p, c_double]),
    "nb2_comm_abort": (c_int, [c_void_p]),
    "nb2_selftest_comm_watchdog": (c_int, [c_int, c_int, c_int, c_double, POINTER(c_int)]),
    "nb2_selftest_peer_wait": (c_int, [c_void_p, c_int64, c_void_p]),
    "nb2_selftest_comm_group": (c_int, [POINTER(c_void_p), c_int, c_int64]),
    "nb2_step_create": (c_int, [POINTER(c_void_p), c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_double]),
    "nb2_step_destroy": (c_int, [c_void_p]),
    "nb2_step_run": (c_int, [c_void_p] * 8 + [c_void_p]),
    "nb2_step_finish": (c_int, [c_void_p, c_void_p]),
}

_lib = None


class Nb2Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libnott_b200 status {status}: {message}")
        self.status = status


def lib() -> ctypes.CDLL:
    """Load libnott_b200.so (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m thot_b200._build` "
                "(this package has no CPU fallback)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise Nb2Error(status, lib().nb2_last_error_string().decode())


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise TypeError(f"libnott_b200 supports float32 and bfloat16, not {dt}")


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise ValueError("libnott_b200 works on CUDA tensors only (no CPU fallback)")


def device_status(clear: bool = True) -> int:
    """Synchronising read of the device status word; raises Nb2Error if a kernel gave up waiting."""
    word = ctypes.c_uint(0)
    check(lib().nb2_device_status(ctypes.byref(word), int(clear)))
    return int(word.value)


def workspace_bytes(op: int, a: int, b: int, dtype: int = F32) -> int:
    return int(lib().nb2_workspace_bytes(op, a, b, dtype))


# --------------------------------------------------------------- norm + act
def layernorm_fwd(x, gamma, beta, eps: float, act: int = ACT_NONE, want_stats: bool = True):
    """x [rows, D] contiguous -> (y, mean, rstd)."""
    _dev(x)
    rows, D = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    check(lib().nb2_layernorm_fwd(_p(x), _p(gamma), _p(beta), _p(y), _p(mean), _p(rstd), rows, D, eps,
                                  dtype_code(x.dtype), act, _stream()))
    return y, mean, rstd


def layernorm_bwd(x, dy, gamma, beta, mean, rstd, act: int = ACT_NONE, want_param_grads: bool = True):
    """-> (dx, dgamma_dbeta [2, D] fp32 or None)."""
    _dev(x)
    rows, D = x.shape
    dx = torch.empty_like(x)
    code = dtype_code(x.dtype)
    partials, out = None, None
    n = c_int64(0)
    if want_param_grads:
        ws = workspace_bytes(WS_NORM_BWD, rows, D, code)
        partials = torch.empty(ws // 4, dtype=torch.float32, device=x.device)
    check(lib().nb2_layernorm_bwd(_p(x), _p(dy), _p(gamma), _p(beta), _p(mean), _p(rstd), _p(dx), _p(partials),
                                  ctypes.byref(n), rows, D, code, act, _stream()))
    if want_param_grads:
        out = torch.empty(2, D, dtype=torch.float32, device=x.device)
        if rows == 0:
            out.zero_()
        else:
            check(lib().nb2_colreduce_partials(_p(partials), n.value, 2 * D, _p(out), _stream()))
    return dx, out


def rmsnorm_fwd(x, weight, eps: float, act: int = ACT_NONE, want_stats: bool = True):
    _dev(x)
    rows, D = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    check(lib().nb2_rmsnorm_fwd(_p(x), _p(weight), _p(y), _p(rstd), rows, D, eps, dtype_code(x.dtype), act, _stream()))
    return y, rstd


def rmsnorm_bwd(x, dy, weight, rstd, act: int = ACT_NONE, want_param_grads: bool = True):
    """-> (dx, dweight [D] fp32 or None)."""
    _dev(x)
    rows, D = x.shape
    dx = torch.empty_like(x)
    code = dtype_code(x.dtype)
    partials, out = None, None
    n = c_int64(0)
    if want_param_grads:
        ws = workspace_bytes(WS_NORM_BWD, rows, D, code)
        partials = torch.empty(ws // 4, dtype=torch.float32, device=x.device)
    check(lib().nb2_rmsnorm_bwd(_p(x), _p(dy), _p(weight), _p(rstd), _p(dx), _p(partials), ctypes.byref(n),
                                rows, D, code, act, _stream()))
    if want_param_grads:
        out = torch.empty(D, dtype=torch.float32, device=x.device)
        if rows == 0:
            out.zero_()
        else:
            check(lib().nb2_colreduce_partials(_p(partials), n.value, D, _p(out), _stream()))
    return dx, out


# ------------------------------------------------------- residual add + norm
def add_norm_fwd(kind, a, b, gamma, beta, eps: float):
    """-> (sum, y, mean or None, rstd): y = norm(a + b), sum = a + b."""
    _dev(a)
    rows, D = a.shape
    s, y = torch.empty_like(a), torch.empty_like(a)
    rstd = torch.empty(rows, dtype=torch.float32, device=a.device)
    if kind == "ln":
        mean = torch.empty(rows, dtype=torch.float32, device=a.device)
        check(lib().nb2_add_layernorm_fwd(_p(a), _p(b), _p(gamma), _p(beta), _p(s), _p(y), _p(mean), _p(rstd), rows, D, eps,
                                          dtype_code(a.dtype), _stream()))
        return s, y, mean, rstd
    check(lib().nb2_add_rmsnorm_fwd(_p(a), _p(b), _p(gamma), _p(s), _p(y), _p(rstd), rows, D, eps, dtype_code(a.dtype), _stream()))
    return s, y, None, rstd


def add_norm_bwd(kind, s, dy, dsum, gamma, mean, rstd):
    """-> (dx, parameter gradients fp32: [2, D] for "ln", [D] for "rms")."""
    _dev(s)
    rows, D = s.shape
    code = dtype_code(s.dtype)
    dx = torch.empty_like(s)
    partials = torch.empty(workspace_bytes(WS_NORM_BWD, rows, D, code) // 4, dtype=torch.float32, device=s.device)
    n = c_int64(0)
    if kind == "ln":
        check(lib().nb2_add_layernorm_bwd(_p(s), _p(dy), _p(dsum), _p(gamma), _p(mean), _p(rstd), _p(dx), _p(partials),
                                          ctypes.byref(n), rows, D, code, _stream()))
        out = torch.empty(2, D, dtype=torch.float32, device=s.device)
    else:
        check(lib().nb2_add_rmsnorm_bwd(_p(s), _p(dy), _p(dsum), _p(gamma), _p(rstd), _p(dx), _p(partials), ctypes.byref(n),
                                        rows, D, code, _stream()))
        out = torch.empty(D, dtype=torch.float32, device=s.device)
    if rows == 0:
        out.zero_()
    else:
        check(lib().nb2_colreduce_partials(_p(partials), n.value, out.numel(), _p(out), _stream()))
    return dx, out


# -------------------------------------------------------------- activations
def act_fwd(x, act: int):
    _dev(x)
    y = torch.empty_like(x)
    check(lib().nb2_act_fwd(_p(x), _p(y), x.numel(), dtype_code(x.dtype), act, _stream()))
    return y


def act_bwd(x, dy, act: int):
    _dev(x)
    dx = torch.empty_like(x)
    check(lib().nb2_act_bwd(_p(x), _p(dy), _p(dx), x.numel(), dtype_code(x.dtype), act, _stream()))
    return dx


def _ld(t):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("silu gate operands must be 2-D with unit column stride")
    return t.stride(0)


def silu_gate_fwd(a, b):
    """out = silu(a) * b; a, b may be row-strided views (halves of a [rows, 2H] tensor)."""
    _dev(a)
    rows, H = a.shape
    out = torch.empty(rows, H, dtype=a.dtype, device=a.device)
    check(lib().nb2_silu_gate_fwd(_p(a), _ld(a), _p(b), _ld(b), _p(out), H, rows, H, dtype_code(a.dtype), _stream()))
    return out


def silu_gate_bwd(a, b, dy, da=None, db=None):
    _dev(a)
    rows, H = a.shape
    if da is None:
        da = torch.empty(rows, H, dtype=a.dtype, device=a.device)
    if db is None:
        db = torch.empty(rows, H, dtype=a.dtype, device=a.device)
    check(lib().nb2_silu_gate_bwd(_p(a), _ld(a), _p(b), _ld(b), _p(dy), _ld(dy), _p(da), _ld(da), _p(db), _ld(db),
                                  rows, H, dtype_code(a.dtype), _stream()))
    return da, db


# ---------------------------------------------------------------- embedding
def _index_code(ids):
    if ids.dtype == torch.int32:
        return I32
    if ids.dtype == torch.int64:
        return I64
    raise TypeError(f"token ids must be int32 or int64, not {ids.dtype}")


def embedding_fwd(table, ids, status=None):
    _dev(table)
    vocab, D = table.shape
    flat = ids.reshape(-1)
    out = torch.empty(flat.numel(), D, dtype=table.dtype, device=table.device)
    check(lib().nb2_embedding_fwd(_p(table), _p(flat), _p(out), flat.numel(), vocab, D, dtype_code(table.dtype),
                                  _index_code(ids), _p(status), _stream()))
    return out.view(*ids.shape, D)


def embedding_bwd(dout, ids, vocab: int):
    _dev(dout)
    D = dout.shape[-1]
    flat = ids.reshape(-1)
    d2 = dout.reshape(-1, D)
    dtable = torch.empty(vocab, D, dtype=dout.dtype, device=dout.device)
    ws_bytes = workspace_bytes(WS_EMBEDDING_BWD, flat.numel(), vocab, dtype_code(dout.dtype))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dout.device)
    check(lib().nb2_embedding_bwd(_p(d2), _p(flat), _p(dtable), flat.numel(), vocab, D, dtype_code(dout.dtype),
                                  _index_code(ids), _p(ws), ws_bytes, _stream()))
    return dtable


def embedding_index(ids, vocab: int, dtype=torch.float32):
    """Sorted token runs of `ids` for embedding_bwd_indexed: build once per ids tensor."""
    flat = ids.reshape(-1).contiguous()
    ws_bytes = workspace_bytes(WS_EMBEDDING_BWD, flat.numel(), vocab, dtype_code(dtype))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=ids.device)
    check(lib().nb2_embedding_index(_p(flat), flat.numel(), vocab, _index_code(ids), _p(ws), ws_bytes, _stream()))
    return ws


def embedding_bwd_indexed(dout, index_ws, vocab: int):
    _dev(dout)
    D = dout.shape[-1]
    d2 = dout.reshape(-1, D)
    dtable = torch.empty(vocab, D, dtype=dout.dtype, device=dout.device)
    check(lib().nb2_embedding_bwd_indexed(_p(d2), _p(dtable), d2.shape[0], vocab, D, dtype_code(dout.dtype), _p(index_ws),
                                          index_ws.numel(), _stream()))
    return dtable


def bert_embedding_ln_fwd(word, pos, type_table, ids, gamma, beta, eps: float = 1e-12, want_backward: bool = True, status=None):
    """ids [B, S] -> (y [B, S, D], sum or None, mean or None, rstd or None)."""
    _dev(word)
    B, S = ids.shape
    vocab, D = word.shape
    y = torch.empty(B, S, D, dtype=word.dtype, device=word.device)
    ssum = torch.empty(B * S, D, dtype=word.dtype, device=word.device) if want_backward else None
    mean = torch.empty(B * S, dtype=torch.float32, device=word.device) if want_backward else None
    rstd = torch.empty(B * S, dtype=torch.float32, device=word.device) if want_backward else None
    check(lib().nb2_bert_embedding_ln_fwd(_p(word), _p(pos), _p(type_table), _p(ids.contiguous()), _p(gamma), _p(beta), _p(ssum),
                                          _p(y), _p(mean), _p(rstd), B, S, vocab, D, eps, dtype_code(word.dtype),
                                          _index_code(ids), _p(status), _stream()))
    return y, ssum, mean, rstd


def bert_embedding_ln_bwd(ssum, dy, ids, gamma, mean, rstd, vocab: int, pos_rows: int = 0, want_type: bool = True):
    """-> (dword [vocab, D], dpos [pos_rows, D] or None, dtype0 [D] or None, dgamma_dbeta [2, D] fp32,
    dsum [B*S, D]: the gradient of the pre-norm sum, from which the three table gradients are formed)."""
    _dev(ssum)
    B, S = ids.shape
    D = ssum.shape[-1]
    code = dtype_code(ssum.dtype)
    dsum = torch.empty_like(ssum)
    dword = torch.empty(vocab, D, dtype=ssum.dtype, device=ssum.device)
    dpos = torch.empty(pos_rows, D, dtype=ssum.dtype, device=ssum.device) if pos_rows else None
    dtype0 = torch.empty(D, dtype=ssum.dtype, device=ssum.device) if want_type else None
    grads = torch.empty(2, D, dtype=torch.float32, device=ssum.device)
    ws_bytes = workspace_bytes(WS_BERT_EMBEDDING_BWD, (B << 32) | S, (vocab << 32) | D, code)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=ssum.device)
    check(lib().nb2_bert_embedding_ln_bwd(_p(ssum), _p(dy.reshape(B * S, D)), _p(ids.contiguous()), _p(gamma), _p(mean), _p(rstd),
                                          _p(dsum), _p(dword), _p(dpos), pos_rows, _p(dtype0), _p(grads), B, S, vocab, D, code,
                                          _index_code(ids), _p(ws), ws_bytes, _stream()))
    return dword, dpos, dtype0, grads, dsum


# ------------------------------------------------------------------ attention
def attention_softmax_fwd(scores, scale: float, key_padding=None, attn_mask=None, causal: bool = False, noise=None,
                          want_pre: bool = True):
    """scores [B, H, T, S] -> attn.  key_padding [B, S] bool/uint8; attn_mask additive, [T,S], [B,T,S],
    [B*H,T,S] or [B,H,T,S] of the scores' dtype.  With `noise` ([B,H,T,S], the dropout's multiplicative
    noise) returns (attn * noise, attn before the noise or None)."""
    _dev(scores)
    B, H, T, S = scores.shape
    out = torch.empty_like(scores)
    sb = sh = 0
    if attn_mask is not None:
        attn_mask = attn_mask.to(scores.dtype).contiguous()
        if attn_mask.dim() == 3 and attn_mask.shape[0] == B:
            sb = T * S
        elif attn_mask.dim() == 4 or (attn_mask.dim() == 3 and attn_mask.shape[0] == B * H):
            sb, sh = H * T * S, T * S
        elif attn_mask.dim() != 2:
            raise ValueError("attention mask must be [T,S], [B,T,S], [B*H,T,S] or [B,H,T,S]")
    if key_padding is not None:
        key_padding = key_padding.to(torch.uint8).contiguous()
    if noise is not None:
        pre = torch.empty_like(scores) if want_pre else None
        check(lib().nb2_attention_softmax_dropout_fwd(_p(scores), _p(key_padding), _p(attn_mask), sb, sh, _p(noise.contiguous()), _p(pre),
                                                      _p(out), B, H, T, S, scale, int(causal), dtype_code(scores.dtype), _stream()))
        return out, pre
    check(lib().nb2_attention_softmax_fwd(_p(scores), _p(key_padding), _p(attn_mask), sb, sh, _p(out), B, H, T, S, scale,
                                          int(causal), dtype_code(scores.dtype), _stream()))
    return out


def attention_softmax_bwd(attn, dattn, scale: float, noise=None):
    """noise given: `attn` is the probabilities before the noise and `dattn` the gradient of attn * noise."""
    _dev(attn)
    S = attn.shape[-1]
    out = torch.empty_like(attn)
    if noise is not None:
        check(lib().nb2_attention_softmax_dropout_bwd(_p(attn), _p(noise.contiguous()), _p(dattn), _p(out), attn.numel() // max(S, 1), S,
                                                      scale, dtype_code(attn.dtype), _stream()))
        return out
    check(lib().nb2_attention_softmax_bwd(_p(attn), _p(dattn), _p(out), attn.numel() // max(S, 1), S, scale,
                                          dtype_code(attn.dtype), _stream()))
    return out


# ------------------------------------------------------------------- linear
_linear_ws = {}


def linear_available() -> bool:
    """Is libnott_b200_linear.so (the tensor-core linear kernels) installed next to the core library?"""
    return bool(lib().nb2_linear_available())


def linear_bias_act_fwd(x, weight, bias=None, act: int = ACT_NONE, want_z: bool = False):
    """y = act(x @ weight.T + bias) on the tensor cores (bf16).  x [M, K], weight [N, K] (torch.nn.Linear's layout),
    bias [N] or None -> (y [M, N], z [M, N] or None)."""
    _dev(x)
    M, K = x.shape
    N = weight.shape[0]
    y = torch.empty(M, N, dtype=x.dtype, device=x.device)
    z = torch.empty(M, N, dtype=x.dtype, device=x.device) if want_z else None
    key = (x.device.index, )
    ws = _linear_ws.get(key)
    if ws is None:
        ws = _linear_ws[key] = torch.empty(workspace_bytes(WS_LINEAR, 0, 0, BF16), dtype=torch.uint8, device=x.device)
    check(lib().nb2_linear_bias_act_fwd(_p(x), _p(weight), _p(bias), _p(z), _p(y), M, N, K, dtype_code(x.dtype), act, _p(ws), ws.numel(),
                                        _stream()))
    return y, z


# --------------------------------------------------------------------- rope
def rope_table(S: int, hd: int, theta: float = 10000.0, positions=None, device="cuda"):
    cs = torch.empty(S, hd // 2, 2, dtype=torch.float32, device=device)
    check(lib().nb2_rope_table(_p(cs), _p(positions), S, hd, theta, _stream()))
    return cs


def rope_apply(x, cos_sin, inverse: bool = False):
    """x [B, S, H, hd] contiguous."""
    _dev(x)
    B, S, H, hd = x.shape
    out = torch.empty_like(x)
    check(lib().nb2_rope_apply(_p(x), _p(cos_sin), _p(out), B, S, H, hd, dtype_code(x.dtype), int(inverse), _stream()))
    return out


# ------------------------------------------------------ host-buffer pipeline
class HostStep:
    """Fused LayerNorm->activation fwd+bwd on HOST buffers (pinned tensors)."""

    def __init__(self, max_rows: int, D: int, dtype: torch.dtype = torch.float32, chunk_rows: int = 0):
        self._ctx = c_void_p()
        self.D, self.dtype = D, dtype
        check(lib().nb2_host_ctx_create(ctypes.byref(self._ctx), max_rows, D, dtype_code(dtype), chunk_rows))

    def step(self, x, dy, gamma, beta, y, dx, dgamma_dbeta, eps: float, act: int):
        for t in (x, dy, gamma, beta, y, dx, dgamma_dbeta):
            if t.is_cuda:
                raise ValueError("HostStep takes host tensors")
        rows = x.shape[0]
        check(lib().nb2_layernorm_act_step_host(self._ctx, _p(x), _p(dy), _p(gamma), _p(beta), _p(y), _p(dx),
                                                _p(dgamma_dbeta), rows, self.D, eps, dtype_code(self.dtype), act))

    def step_rms(self, x, dy, weight, y, dx, dweight, eps: float, act: int):
        for t in (x, dy, weight, y, dx, dweight):
            if t.is_cuda:
                raise ValueError("HostStep takes host tensors")
        rows = x.shape[0]
        check(lib().nb2_rmsnorm_act_step_host(self._ctx, _p(x), _p(dy), _p(weight), _p(y), _p(dx), _p(dweight), rows, self.D, eps,
                                              dtype_code(self.dtype), act))

    def close(self):
        if self._ctx:
            lib().nb2_host_ctx_destroy(self._ctx)
            self._ctx = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------- row-sharded step
def comm_unique_id() -> bytes:
    """Rank 0 makes the id; the other ranks receive it over any host-side channel."""
    buf = ctypes.create_string_buffer(COMM_ID_BYTES)
    check(lib().nb2_comm_unique_id(buf))
    return buf.raw


class Comm:
    """One communicator per process (device = torch's current device)."""

    def __init__(self, unique_id, rank: int, world: int, exchange: int = EXCHANGE_NCCL, max_cols: int = 2 * 8192):
        self._h = c_void_p()
        self.rank, self.world, self.exchange = rank, world, exchange
        idbuf = ctypes.create_string_buffer(bytes(unique_id), COMM_ID_BYTES) if unique_id is not None else None
        check(lib().nb2_comm_create(ctypes.byref(self._h), idbuf, rank, world, exchange, max_cols))

    @property
    def handle(self):
        return self._h

    def exchange_begin(self, partials, n_partials: int, grads):
        check(lib().nb2_grad_exchange_begin(self._h, _p(partials), n_partials, grads.numel(), _p(grads), _stream()))

    def exchange_end(self):
        check(lib().nb2_grad_exchange_end(self._h, _stream()))

    def allreduce_(self, grads):
        """In-place sum over ranks of one fp32 vector (a single "partial")."""
        src = grads.clone()
        self.exchange_begin(src, 1, grads)
        self.exchange_end()
        return grads

    def wait(self, timeout_s: float):
        check(lib().nb2_comm_wait(self._h, float(timeout_s)))

    def abort(self):
        check(lib().nb2_comm_abort(self._h))

    def close(self):
        if self._h:
            lib().nb2_comm_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def attention_softmax_order(order: int) -> int:
    """0 by size, 1 memory order, 2 heads innermost whenever the mask is shared by the heads -> the previous setting."""
    before = lib().nb2_attention_softmax_order(order)
    if before < 0:
        check(before)
    return before


def comm_group(world: int, max_cols: int):
    """`world` linked peer-form communicators on the current device (see nb2_selftest_comm_group): a list of Comm."""
    arr = (c_void_p * world)()
    check(lib().nb2_selftest_comm_group(arr, world, max_cols))
    out = []
    for r in range(world):
        c = Comm.__new__(Comm)
        c._h, c.rank, c.world, c.exchange = c_void_p(arr[r]), r, world, EXCHANGE_PEER
        out.append(c)
    return out


class NormStep:
    """forward + backward + partial reduce + exchange of one norm layer on this rank's rows."""

    def __init__(self, comm, kind: str, rows: int, D: int, dtype: torch.dtype, act: int, eps: float):
        self._h = c_void_p()
        self._comm = comm          # keeps the communicator alive
        self.kind, self.rows, self.D = kind, rows, D
        check(lib().nb2_step_create(ctypes.byref(self._h), comm.handle if comm is not None else None,
                                    NORM_LAYER if kind == "ln" else NORM_RMS, rows, D, dtype_code(dtype), act, eps))

    def run(self, x, dy, gamma, beta, y, dx, grads):
        check(lib().nb2_step_run(self._h, _p(x), _p(dy), _p(gamma), _p(beta), _p(y), _p(dx), _p(grads), _stream()))

    def finish(self):
        check(lib().nb2_step_finish(self._h, _stream()))

    def close(self):
        if self._h:
            lib().nb2_step_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
