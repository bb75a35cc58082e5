"""The binding harness on CPU: the reference's own RegisteredLayer running its unfused pair
(torch::nn::LayerNorm bound with bind_module_forward, then apply(GeLU)) agrees with the C restatement,
and an empty ForwardBinding raises as registry.hpp:44-46 says.  The CUDA half is in
tests/test_gpu_reference_binding.py."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import cpu_oracle as O
from oracle import reference as R
from tests import tol

pytestmark = pytest.mark.skipif(not R.binding_available(), reason="oracle/_ref/libnott_binding.so not built (needs the reference checkout)")


def test_reference_pair_through_registered_layer_matches_the_oracle():
    rng = np.random.default_rng(3)
    B, S, D = 2, 9, 256
    x = rng.standard_normal((B, S, D)).astype(np.float32); dy = rng.standard_normal((B, S, D)).astype(np.float32)
    g = (1 + 0.02 * rng.standard_normal(D)).astype(np.float32); b = (0.02 * rng.standard_normal(D)).astype(np.float32)
    ref = O.layernorm_act(x.reshape(-1, D), g, b, dy.reshape(-1, D), 1e-5, O.ACT_GELU)
    r64 = R.binding_layernorm_gelu(R.BIND_REFERENCE_F64, x, dy, g, b)
    r32 = R.binding_layernorm_gelu(R.BIND_REFERENCE_F32, x, dy, g, b)
    for got in (r64, r32):
        tol.fp32_close(got["y"].reshape(-1, D), ref["y"], rtol=1e-5, atol=2e-6)
        tol.fp32_close(got["dx"].reshape(-1, D), ref["dx"], rtol=1e-5, atol=2e-6)
        tol.long_sum_close(got["dgamma"], ref["dgamma"], B * S)
        tol.long_sum_close(got["dbeta"], ref["dbeta"], B * S)


def test_empty_binding_raises_logic_error():
    assert R.binding_lib().refbind_empty_binding_raises() == 1
