"""Row a8 of the scope: the reference's own layer binding drives the drop-in module.
A Nott::B200::LayerNorm with GeLU fused is bound through RegisteredLayer::bind_module_forward
(src/layer/registry.hpp:51-57), layer.activation is Identity, and the pair
`layer.forward(x)` -> `apply(layer.activation, .)` of src/core.hpp:1927-1934 runs on a CUDA tensor; also through
a copy of the layer and through an inline-functor binding that is copied, moved and assigned (the context
re-pointing of registry.hpp:157-168).  Compared with the unfused reference pair (torch::nn::LayerNorm +
apply(GeLU)) run through the same RegisteredLayer on CPU, forward and backward."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import cpu_oracle as O
from oracle import reference as R
from tests import tol

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not R.binding_available(), reason="oracle/_ref/libnott_binding.so not built (needs the reference checkout)")]


@pytest.mark.parametrize("which", [R.BIND_MODULE, R.BIND_COPY, R.BIND_INLINE_COPY_MOVE])
@pytest.mark.parametrize("B,S,D", [(4, 64, 1024), (2, 33, 768), (3, 5, 100)])
def test_registered_layer_runs_the_fused_module_like_the_reference_pair(which, B, S, D):
    rng = np.random.default_rng(B * 1000 + D)
    x = rng.standard_normal((B, S, D)).astype(np.float32); dy = rng.standard_normal((B, S, D)).astype(np.float32)
    g = (1 + 0.02 * rng.standard_normal(D)).astype(np.float32); b = (0.02 * rng.standard_normal(D)).astype(np.float32)
    got = R.binding_layernorm_gelu(which, x, dy, g, b)
    r32 = R.binding_layernorm_gelu(R.BIND_REFERENCE_F32, x, dy, g, b)
    r64 = R.binding_layernorm_gelu(R.BIND_REFERENCE_F64, x, dy, g, b)
    ref = O.layernorm_act(x.reshape(-1, D), g, b, dy.reshape(-1, D), 1e-5, O.ACT_GELU)      # fp64 arbiter for y and dx
    tol.fp32_close_adjudicated(got["y"].reshape(-1, D), r32["y"].reshape(-1, D), ref["y"])
    tol.fp32_close_adjudicated(got["dx"].reshape(-1, D), r32["dx"].reshape(-1, D), ref["dx"])
    tol.long_sum_close(got["dgamma"], ref["dgamma"], B * S, ref32=r32["dgamma"], strict=True, label=f"a8 binding {which} D={D} dgamma")
    tol.long_sum_close(got["dbeta"], ref["dbeta"], B * S, ref32=r32["dbeta"], strict=True, label=f"a8 binding {which} D={D} dbeta")
    np.testing.assert_allclose(r64["dgamma"], ref["dgamma"], rtol=1e-5, atol=1e-5)


def test_bf16_module_through_the_binding():
    rng = np.random.default_rng(9)
    B, S, D = 2, 40, 2048
    x = rng.standard_normal((B, S, D)).astype(np.float32); dy = rng.standard_normal((B, S, D)).astype(np.float32)
    g = (1 + 0.02 * rng.standard_normal(D)).astype(np.float32); b = (0.02 * rng.standard_normal(D)).astype(np.float32)
    rb = lambda a: tol.bf16_bits_to_f32(tol.to_bf16_bits(a)).reshape(a.shape)  # noqa: E731
    xb, dyb, gb, bb = rb(x), rb(dy), rb(g), rb(b)
    got = R.binding_layernorm_gelu(R.BIND_MODULE, xb, dyb, gb, bb, bf16=True)
    ref = O.layernorm_act(xb.reshape(-1, D), gb, bb, dyb.reshape(-1, D), 1e-5, O.ACT_GELU)
    tol.bf16_ulp_close(tol.to_bf16_bits(got["y"].reshape(-1, D)), ref["y"])
    tol.bf16_ulp_close(tol.to_bf16_bits(got["dx"].reshape(-1, D)), ref["dx"])
