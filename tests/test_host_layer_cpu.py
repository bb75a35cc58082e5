"""Host-side behaviour of the C++ layer that needs no GPU: the binding loads, options are
validated with the reference's exception types, and nothing falls back to the CPU."""
from __future__ import annotations

import pytest
import torch


@pytest.fixture(scope="module")
def host():
    from thot_b200 import _nott_b200_host as h
    return h


def test_constructor_and_input_errors_match_the_reference_messages(host):
    msgs = host.module_errors()
    # Mamba RMSNorm's own messages (src/block/details/transformers/mamba.hpp:116-128)
    assert msgs[0] == "RMSNorm requires a positive embedding dimension."
    assert msgs[1] == "RMSNorm requires a defined input tensor."
    assert "no CPU fallback" in msgs[2]


def test_cpu_tensors_are_refused_not_computed(host):
    x = torch.randn(4, 64)
    for call in (lambda: host.layernorm_act(x, None, None, 1e-5, 0),
                 lambda: host.rmsnorm_act(x, None, 1e-6, 0),
                 lambda: host.apply(7, x),
                 lambda: host.silu_gate(x, x),
                 lambda: host.embedding(x, torch.zeros(3, dtype=torch.long))):
        with pytest.raises(ValueError):
            call()


def test_apply_covers_only_the_path_activations(host):
    x = torch.randn(4)
    assert torch.equal(host.apply(0, x), x)          # Identity returns its input, as the reference does
    for other in (1, 2, 3, 4, 5, 8, 10, 11, 12):     # ReLU .. Mish: not on this path
        with pytest.raises(ValueError):
            host.apply(other, x)
