"""bench.py's host-side logic that needs no GPU: workload parsing, algorithmic byte counts and the
argument validation of the C ABI calls it relies on (validation returns before any device work)."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_default_workload_is_the_sweep_point_in_the_target_range(bench):
    w = bench.Workload(bench.DEFAULT_WORKLOAD, 8)
    assert (w.kind, w.dtype, w.D, w.rows_per_rank, w.scaling) == ("ln", torch.float32, 2048, (1 << 20) // 8, "strong")
    one = bench.Workload(bench.DEFAULT_WORKLOAD, 1)
    assert bench.config_of(one, 1)["global_rows"] == bench.config_of(w, 8)["global_rows"] == 1 << 20
    assert set(bench.config_of(one, 1)) == {"workload", "workload_spec", "rows_per_gpu", "D", "global_rows", "l2"}


def test_cfg2_workload_is_the_fp32_layernorm_gelu_case(bench):
    w = bench.Workload("cfg2", 8)
    assert (w.kind, w.dtype, w.D, w.rows_per_rank, w.scaling) == ("ln", torch.float32, 1024, 32768, "weak")
    n, d = 32768, 1024
    assert w.fwd_bytes() == 2 * n * d * 4 + 8 * n + 2 * d * 4
    assert w.bwd_bytes() == 3 * n * d * 4 + 8 * n + 2 * d * 8


def test_sweep_workloads_split_rows_and_accept_a_reduced_row_count(bench):
    w = bench.Workload("cfg5:rms:bf16:4096", 8)
    assert (w.kind, w.dtype, w.D, w.rows_per_rank, w.scaling, w.act) == ("rms", torch.bfloat16, 4096, (1 << 20) // 8, "strong", 2)
    small = bench.Workload("cfg5:ln:bf16:1024:131072", 1)
    assert small.rows_per_rank == 131072 and "reduced row count" in small.name
    with pytest.raises(SystemExit):
        bench.Workload("cfg5:ln:fp32:1024", 3)            # 2^20 rows do not split over 3 ranks
    with pytest.raises(SystemExit):
        bench.Workload("cfg9", 1)


def test_abi_argument_checks_return_before_touching_a_device():
    from thot_b200 import abi
    L = abi.lib()
    assert L.nb2_attention_softmax_fwd(None, None, None, 0, 0, None, 1, 1, 1, 8, 1.0, 0, 9, None) == -3      # dtype
    assert L.nb2_attention_softmax_fwd(None, None, None, 0, 0, None, 1, 1, -1, 8, 1.0, 0, 0, None) == -2     # shape
    assert L.nb2_attention_softmax_bwd(None, None, None, 0, 8, 1.0, 0, None) == 0                            # empty
    assert L.nb2_embedding_index(None, 5, 0, 0, None, 0, None) == -2                                         # vocab
    assert L.nb2_embedding_index(None, 0, 10, 0, None, 0, None) == 0                                         # no tokens
    assert L.nb2_selftest_bounded_wait(0, None, None) == -2
    assert b"cycle_limit" in L.nb2_last_error_string()


def test_reference_arm_prints_the_same_config_and_the_requested_steps(bench):
    """`bench.py --impl reference` needs no GPU: one JSON line with the GPU arm's metric, unit and config object, the
    requested steps and warm-up, an e2e object that repeats the value with zero copy bytes, and a cpu_baseline record."""
    import json
    import subprocess
    from oracle import reference as R
    if not R.available():
        pytest.skip("oracle/_ref/libnott_ref.so not built (needs the reference checkout)")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
                          "--workload", "cfg5:ln:fp32:1024:4096"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == bench.UNIT
    assert (line["steps"], line["warmup"], line["n_gpus"], line["higher_is_better"]) == (2, 1, 1, True)
    assert line["config"] == bench.config_of(bench.Workload("cfg5:ln:fp32:1024:4096", 1), 1)
    assert line["e2e"] == {"value": line["value"], "unit": bench.UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] >= 1 and line["gpu_launches"] == 0
