"""Row sharding + the one allreduce, world_size 2 over gloo on CPU.  The per-rank
arithmetic is the CPU oracle (there is no GPU here); what is under test is the
partition and the exchange in thot_b200/sharding.py."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from thot_b200.sharding import ExchangeError, allreduce_param_grads, check_layout, row_shard


def test_row_shard_partitions_exactly():
    for rows in (0, 1, 7, 8, 1 << 20, (1 << 20) + 5):
        for world in (1, 2, 3, 4, 8):
            spans = [row_shard(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0
            assert sum(c for _, c in spans) == rows
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        row_shard(10, 2, 2)


def test_allreduce_is_noop_without_process_group():
    g = torch.arange(6, dtype=torch.float32)
    assert torch.equal(allreduce_param_grads(g.clone()), g)
    with pytest.raises(TypeError):
        allreduce_param_grads(torch.zeros(3, dtype=torch.float64))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, D, result_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import cpu_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(123)                      # every rank builds the same global tensors
        x = rng.standard_normal((rows, D)).astype(np.float32)
        dy = rng.standard_normal((rows, D)).astype(np.float32)
        gamma = (1 + 0.02 * rng.standard_normal(D)).astype(np.float32)
        beta = (0.02 * rng.standard_normal(D)).astype(np.float32)
        start, count = row_shard(rows, world, rank)
        part = O.layernorm_act(x[start:start + count], gamma, beta, dy[start:start + count], 1e-5, O.ACT_GELU)
        grads = torch.from_numpy(np.stack([part["dgamma"], part["dbeta"]]).astype(np.float32))
        allreduce_param_grads(grads)
        full = O.layernorm_act(x, gamma, beta, dy, 1e-5, O.ACT_GELU)
        ref = np.stack([full["dgamma"], full["dbeta"]])
        np.testing.assert_allclose(grads.numpy(), ref, rtol=1e-5, atol=1e-5)
        # dX and y of the shard are exactly the corresponding rows of the full run
        np.testing.assert_array_equal(part["dx"], full["dx"][start:start + count])
        np.testing.assert_array_equal(part["y"], full["y"][start:start + count])
        with open(os.path.join(result_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows", [37, 64])
def test_two_rank_gloo_allreduce_matches_unsharded(tmp_path, rows):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, rows, 48, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


# ---- failures made on the host: a rank with another D, a rank that never joins the exchange
def _mismatch_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D = 48 if rank == 0 else 64                      # rank 1 was configured with another width
        try:
            check_layout(2 * D, "ln", 0, timeout_s=20.0)
        except ExchangeError as exc:
            assert "disagree" in str(exc)
            with open(os.path.join(result_dir, f"raised{rank}"), "w") as f:
                f.write(str(exc))
    finally:
        dist.destroy_process_group()


def test_rank_with_another_width_is_an_error_not_a_hang(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_mismatch_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"raised{r}").exists() for r in range(world))


def _skip_worker(rank, world, port, result_dir):
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.ones(16, dtype=torch.float32)
        allreduce_param_grads(g, timeout_s=20.0)          # step 0: everybody joins
        assert torch.equal(g, torch.full((16,), float(world)))
        if rank == 1:
            time.sleep(3.0)                               # step 1: this rank leaves between steps and never joins
        else:
            t0 = time.perf_counter()
            try:
                allreduce_param_grads(torch.ones(16, dtype=torch.float32), timeout_s=1.0)
            except ExchangeError as exc:
                waited = time.perf_counter() - t0
                with open(os.path.join(result_dir, "raised0"), "w") as f:
                    f.write(f"{waited:.2f} {exc}")
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_that_skips_the_exchange_times_the_others_out(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_skip_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    text = (tmp_path / "raised0").read_text()
    assert float(text.split()[0]) < 2.5, text          # raised at the 1 s deadline, not when the peer left


def test_watchdog_policy_without_a_gpu():
    """nb2_comm_wait's policy against scripted callbacks: completion, an asynchronous error of the
    communicator (abort + NB2_ERR_COMM) and a deadline that passes (abort + NB2_ERR_COMM_TIMEOUT)."""
    import ctypes
    import time
    from thot_b200 import abi
    L = abi.lib()
    aborts = ctypes.c_int(-1)
    assert L.nb2_selftest_comm_watchdog(5, -1, 0, 1.0, ctypes.byref(aborts)) == 0 and aborts.value == 0
    assert L.nb2_selftest_comm_watchdog(-1, 3, 5, 1.0, ctypes.byref(aborts)) == abi.ERR_COMM and aborts.value == 1
    assert b"asynchronous error 5" in L.nb2_last_error_string()
    t0 = time.perf_counter()
    assert L.nb2_selftest_comm_watchdog(-1, -1, 0, 0.2, ctypes.byref(aborts)) == abi.ERR_COMM_TIMEOUT and aborts.value == 1
    assert 0.15 < time.perf_counter() - t0 < 1.0
    # completion that arrives before a later error wins
    assert L.nb2_selftest_comm_watchdog(2, 10, 5, 1.0, ctypes.byref(aborts)) == 0 and aborts.value == 0
