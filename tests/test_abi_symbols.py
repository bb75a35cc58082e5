"""The C-ABI library loads and exports every function include/nott_b200.h declares;
argument validation (host logic, no device needed) returns the documented codes."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from thot_b200 import abi

HEADER = Path(__file__).resolve().parents[1] / "include" / "nott_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(nb2_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("nb2_layernorm_fwd", "nb2_layernorm_bwd", "nb2_colreduce_partials", "nb2_rmsnorm_fwd",
                 "nb2_rmsnorm_bwd", "nb2_act_fwd", "nb2_act_bwd", "nb2_silu_gate_fwd", "nb2_silu_gate_bwd",
                 "nb2_embedding_fwd", "nb2_embedding_bwd", "nb2_rope_table", "nb2_rope_apply",
                 "nb2_workspace_bytes", "nb2_last_error_string", "nb2_layernorm_act_step_host"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = abi.lib()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in nott_b200.h but not exported"
        assert name in abi._SIGNATURES, f"{name} has no ctypes signature in thot_b200/abi.py"
    assert lib.nb2_abi_version() == 1


def test_no_undeclared_exports():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(abi.LIB_PATH)], capture_output=True, text=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    assert exported == set(declared_functions())


def test_argument_validation_codes():
    lib = abi.lib()
    one = ctypes.c_void_p(16)          # never dereferenced: validation fails first
    n = ctypes.c_int64(0)
    # unknown dtype / activation
    assert lib.nb2_layernorm_fwd(one, None, None, one, None, None, 4, 8, 1e-5, 7, 0, None) == -3
    assert lib.nb2_layernorm_fwd(one, None, None, one, None, None, 4, 8, 1e-5, 0, 9, None) == -3
    assert b"activation" in lib.nb2_last_error_string()
    # bad shapes
    assert lib.nb2_layernorm_fwd(one, None, None, one, None, None, 4, 0, 1e-5, 0, 0, None) == -2
    assert lib.nb2_rmsnorm_fwd(one, None, one, None, -1, 8, 1e-6, 0, 0, None) == -2
    assert lib.nb2_rope_table(one, None, 4, 7, 10000.0, None) == -2          # odd head_dim
    assert lib.nb2_silu_gate_fwd(one, 4, one, 8, one, 8, 2, 8, 0, None) == -2   # lda < H
    # NULL pointers
    assert lib.nb2_layernorm_fwd(None, None, None, one, None, None, 4, 8, 1e-5, 0, 0, None) == -1
    assert lib.nb2_layernorm_bwd(one, one, None, None, None, one, one, None, ctypes.byref(n), 4, 8, 0, 0, None) == -1
    assert lib.nb2_embedding_fwd(one, None, one, 3, 10, 8, 0, 0, None, None) == -1
    assert lib.nb2_embedding_fwd(one, one, one, 3, 10, 8, 0, 5, None, None) == -3
    # empty inputs are a no-op, not an error
    assert lib.nb2_layernorm_fwd(None, None, None, None, None, None, 0, 8, 1e-5, 0, 0, None) == 0
    assert lib.nb2_act_fwd(None, None, 0, 1, 1, None) == 0
    assert lib.nb2_silu_gate_fwd(None, 0, None, 0, None, 0, 0, 16, 1, None) == 0
    assert lib.nb2_embedding_fwd(None, None, None, 0, 10, 8, 0, 0, None, None) == 0
    assert lib.nb2_rope_apply(None, None, None, 0, 5, 2, 8, 0, 0, None) == 0


def test_workspace_queries_are_consistent():
    # LayerNorm backward partials: at most one [2, D] fp32 block per persistent CTA
    b = abi.workspace_bytes(abi.WS_NORM_BWD, 32768, 1024, abi.F32)
    assert 2 * 1024 * 4 <= b <= 2 * 1024 * 4 * 148 * 2 + 256
    small = abi.workspace_bytes(abi.WS_NORM_BWD, 3, 1024, abi.F32)
    assert small <= b
    assert abi.workspace_bytes(abi.WS_ROPE_TABLE, 2048, 128) == 2048 * 64 * 2 * 4
    assert abi.workspace_bytes(99, 1, 1) == 0


def test_python_host_refuses_cpu_tensors():
    import torch
    x = torch.zeros(2, 8)
    with pytest.raises(ValueError):
        abi.layernorm_fwd(x, None, None, 1e-5)
    with pytest.raises(TypeError):
        abi.dtype_code(torch.float16)


def test_ctypes_signatures_match_the_header_prototypes():
    """Every binding in thot_b200/abi.py passes exactly as many arguments as the C prototype takes,
    and a pointer where the prototype has a pointer."""
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    protos = re.findall(r"\b(?:int|size_t|const char\*)\s+(nb2_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)
    assert len(protos) == len(declared_functions())
    for name, args in protos:
        params = [a.strip() for a in args.replace("\n", " ").split(",")] if args.strip() != "void" else []
        res, argtypes = abi._SIGNATURES[name]
        assert len(argtypes) == len(params), f"{name}: header has {len(params)} parameters, binding {len(argtypes)}"
        for p, t in zip(params, argtypes):
            is_ptr = "*" in p
            bound_ptr = t in (ctypes.c_void_p, ctypes.c_char_p) or hasattr(t, "contents") or getattr(t, "_type_", None) not in ("i", "l", "q", "d", "L", "Q", "I")
            if is_ptr:
                assert bound_ptr, f"{name}: '{p}' is a pointer but is bound as {t}"
            else:
                assert t in (ctypes.c_int, ctypes.c_int64, ctypes.c_double, ctypes.c_size_t), f"{name}: '{p}' bound as {t}"


def test_reserve_sms_is_a_host_side_setting_that_returns_the_previous_value():
    from thot_b200 import abi
    L = abi.lib()
    before = L.nb2_reserve_sms(3)
    try:
        assert L.nb2_reserve_sms(5) == 3
        assert L.nb2_reserve_sms(-7) == 5          # negative means none
        assert L.nb2_reserve_sms(0) == 0
    finally:
        L.nb2_reserve_sms(before)


def test_softmax_row_order_is_a_host_side_setting_that_returns_the_previous_value():
    from thot_b200 import abi
    L = abi.lib()
    before = L.nb2_attention_softmax_order(1)
    try:
        assert L.nb2_attention_softmax_order(2) == 1
        assert L.nb2_attention_softmax_order(0) == 2
        assert L.nb2_attention_softmax_order(3) == -2 and L.nb2_attention_softmax_order(-1) == -2      # NB2_ERR_SHAPE
        assert L.nb2_attention_softmax_order(0) == 0                                                    # unchanged by the refusals
    finally:
        L.nb2_attention_softmax_order(before)
