#!/usr/bin/env python
"""Benchmark of the fused norm+activation path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg5:<ln|rms>:<fp32|bf16>:<D>[:<rows>]|cfg2] [--exchange nccl|peer]

One step = LayerNorm->GELU (or RMSNorm->SiLU) forward, backward (dX + per-CTA
dgamma/dbeta partials), the partial reduce, and for N > 1 the sum over ranks of
the [2, D] gradients (NCCL allreduce, or the library's own peer-store exchange).
Default workload: one point of the whole-box sweep in the range the metric's
targets are stated for: 2^20 rows x D=2048 fp32, LayerNorm -> exact GELU, eps 1e-5,
rows split evenly over the ranks (strong scaling).  `cfg2` is x[32,1024,1024] fp32
per GPU (weak scaling); the default run also reports it as a sub-record so the
behaviour of a 0.12 ms step stays visible.

Prints ONE JSON line on rank 0.  `value` is algorithmic HBM GB/s of the whole job
(inputs resident in HBM), `e2e` the same metric through the host-buffer C-ABI call
(pinned host buffers, copies inside the timed region), `roofline` the dominant
kernel against the measured HBM peak, `cpu_baseline` the reference's CPU path on
a bounded sample on this box's host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "fused_norm_act_fwd_bwd_hbm_gbs"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0          # used only when MEASURED_PEAKS.json is absent
DEFAULT_WORKLOAD = "cfg5:ln:fp32:2048"


# ----------------------------------------------------------------- workloads
class Workload:
    def __init__(self, spec: str, world: int):
        self.spec = spec
        if spec == "cfg2":
            self.kind, self.dtype, self.D = "ln", torch.float32, 1024
            self.rows_per_rank, self.scaling = 32 * 1024, "weak"
            self.name = "LayerNorm->GELU(erf) fwd+bwd fp32 x[32,1024,1024] per GPU"
        elif spec.startswith("cfg5:"):
            # an optional fifth field shrinks the row count: the same kernels on a case small enough to profile
            parts = spec.split(":")
            kind, dt, D = parts[1:4]
            self.kind, self.D = kind, int(D)
            self.dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dt]
            total = int(parts[4]) if len(parts) > 4 else 1 << 20
            if total % world:
                raise SystemExit(f"cfg5 needs a world size that divides {total}")
            self.rows_per_rank, self.scaling = total // world, "strong"
            rows_txt = "2^20" if total == 1 << 20 else str(total)
            self.name = (f"{'LayerNorm->GELU' if kind == 'ln' else 'RMSNorm->SiLU'} fwd+bwd {dt} {rows_txt} rows x D={D} "
                         + ("(whole-box sweep configuration)" if total == 1 << 20 else "(sweep kernels on a reduced row count)"))
        else:
            raise SystemExit(f"unknown workload {spec}")
        self.act = 1 if self.kind == "ln" else 2          # GELU behind LayerNorm, SiLU behind RMSNorm
        self.eps = 1e-5 if self.kind == "ln" else 1e-6
        self.elt = 4 if self.dtype == torch.float32 else 2

    # algorithmic bytes, per rank
    def fwd_bytes(self, rows=None):
        n = self.rows_per_rank if rows is None else rows
        stats = 8 * n if self.kind == "ln" else 4 * n
        params = (2 if self.kind == "ln" else 1) * self.D * self.elt
        return 2 * n * self.D * self.elt + stats + params

    def bwd_bytes(self, rows=None):
        n = self.rows_per_rank if rows is None else rows
        stats = 8 * n if self.kind == "ln" else 4 * n
        params = (2 if self.kind == "ln" else 1) * self.D * (self.elt + 4)     # read gamma/beta, write fp32 grads
        return 3 * n * self.D * self.elt + stats + params

    def step_bytes(self, rows=None):
        return self.fwd_bytes(rows) + self.bwd_bytes(rows)


def synth_inputs(w: Workload, rows: int, device, seed: int):
    """Synthetic N(0,1) activations, gamma = 1 + N(0,0.02), beta = N(0,0.02)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(rows, w.D, device=device, generator=gen).to(w.dtype)
    dy = torch.randn(rows, w.D, device=device, generator=gen).to(w.dtype)
    gamma = (1 + 0.02 * torch.randn(w.D, device=device, generator=gen)).to(w.dtype)
    beta = (0.02 * torch.randn(w.D, device=device, generator=gen)).to(w.dtype) if w.kind == "ln" else None
    return x, dy, gamma, beta


# -------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls NVML for SM clock and throttle reasons.  The thread is started before the warm-up
    and polls every 20 ms; samples count only while `armed` (the timed region), so nothing is
    created or torn down inside that region."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period_s = period_s
        self.armed = False
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def sample(self):
        if self.nv is None:
            return
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            r = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                     0x4: "sw_power_cap", 0x80: "hw_power_brake"}
            for bit, nm in names.items():
                if r & bit:
                    self.reasons.add(nm)
        except Exception:
            pass

    def start(self):
        def loop():
            while not self._stop.is_set():
                if self.armed:
                    self.sample()
                time.sleep(self.period_s)
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------- reference arm
def config_of(w: Workload, world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": w.name, "workload_spec": w.spec, "rows_per_gpu": w.rows_per_rank, "D": w.D,
            "global_rows": w.rows_per_rank * world,
            "l2": "inputs larger than L2 (each step streams %.0f MB per GPU)" % (w.step_bytes() / 1e6)}


def reference_cpu_run(w: Workload, steps: int, warmup: int, budget_s: float = 20.0, exact_steps: bool = False):
    """The reference's own modules (oracle/_ref: Nott headers + libtorch CPU, all host threads),
    forward + autograd backward, on a bounded row sample of the workload (at most 32 Mi elements);
    timed inside the harness so only the module calls are on the clock.  With `exact_steps` the
    requested number of timed passes is kept and the row sample shrinks to fit the time budget;
    otherwise the number of passes shrinks.  Falls back to the single-core C port when the
    reference library was not built.  Returns (GB/s, seconds per step, sample rows, passes, description)."""
    from oracle import reference as R
    from oracle import cpu_oracle as O

    use_ref = R.available()
    bf16 = w.dtype == torch.bfloat16
    if use_ref:
        R.set_num_threads(os.cpu_count() or 1)      # torchrun exports OMP_NUM_THREADS=1; the baseline gets every host core
        sample_rows = max(1, min(w.rows_per_rank, (32 << 20) // w.D))
        compute = 2 if bf16 else 0       # the reference runs in the tensor's own dtype
        per = R.time_norm_act(w.kind, sample_rows, w.D, w.eps, w.act, compute, iters=1, warmup=1)
        if exact_steps:
            n = max(1, steps)
            total = per * (n + warmup)
            if total > budget_s:
                sample_rows = max(64, int(sample_rows * budget_s / total))
            sec = R.time_norm_act(w.kind, sample_rows, w.D, w.eps, w.act, compute, iters=n, warmup=max(0, warmup))
        else:
            n = max(1, min(steps, int(budget_s / max(per, 1e-6))))
            sec = R.time_norm_act(w.kind, sample_rows, w.D, w.eps, w.act, compute, iters=n, warmup=0)
        cores = R.num_threads()
    else:
        sample_rows = min(w.rows_per_rank, 512)
        rng = np.random.default_rng(0)
        x = rng.standard_normal((sample_rows, w.D)).astype(np.float32)
        dy = rng.standard_normal((sample_rows, w.D)).astype(np.float32)
        gamma = (1 + 0.02 * rng.standard_normal(w.D)).astype(np.float32)
        beta = (0.02 * rng.standard_normal(w.D)).astype(np.float32)

        def one():
            if w.kind == "ln":
                O.layernorm_act(x, gamma, beta, dy, w.eps, w.act)
            else:
                O.rmsnorm_act(x, gamma, dy, w.eps, w.act)

        one()
        t0 = time.perf_counter()
        one()
        per = time.perf_counter() - t0
        n = max(1, steps) if exact_steps and per * steps <= budget_s else max(1, min(steps, int(budget_s / max(per, 1e-6))))
        t0 = time.perf_counter()
        for _ in range(n):
            one()
        sec = (time.perf_counter() - t0) / n
        cores = 1
    gbs = w.step_bytes(sample_rows) / sec / 1e9
    desc = {
        "value": gbs, "unit": UNIT, "cores": cores,
        "kind": "reference" if use_ref else "port",
        "sample": f"{sample_rows} of {w.rows_per_rank} rows x D={w.D}, {n} timed fwd+bwd passes, "
                  + ("Nott modules on libtorch CPU, native " + ("bf16" if bf16 else "fp32") if use_ref
                     else "scalar C restatement in fp64"),
        "rows_per_s": sample_rows / sec, "ms_per_pass": sec * 1e3, "host_cpus": os.cpu_count(),
    }
    return gbs, sec, sample_rows, n, desc


def run_reference_arm(args, w: Workload, rank: int, world: int):
    """`--impl reference`: the reference's CPU implementation of the same step on this box's host
    cores; rank 0 alone runs it.  Same metric, unit, config, steps and warmup as the GPU arm; each
    step is a bounded row sample of the workload."""
    if rank != 0:
        return
    gbs, sec, sample_rows, n, desc = reference_cpu_run(w, args.steps, args.warmup, budget_s=240.0, exact_steps=True)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": world, "steps": n,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": w.scaling,
        "vs_baseline": None, "dtype": "f32" if w.dtype == torch.float32 else "bf16", "data": "synthetic",
        "config": config_of(w, world),
        "note": "reference CPU implementation on the host cores; each step is a bounded row sample (see cpu_baseline.sample)",
        "cpu_baseline": desc,
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "rows_per_s": sample_rows / sec, "gpu_launches": 0,
    }
    _emit(line)


# ---------------------------------------------------------------- op suite
def run_suite(args):
    """`--suite`: every other kernel of the path at the benchmark's RMSNorm/gate and gather/rotary configuration sizes, one launch type per
    entry, CUDA-event timed, algorithmic bytes / time against the measured HBM peak.  One JSON line."""
    from thot_b200 import abi

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_file.read_text())["hbm_gbs"]) if peaks_file.exists() else FALLBACK_HBM_GBS
    results = []

    def timed(name, fn, nbytes, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / iters / 1e3
        results.append({"op": name, "us": sec * 1e6, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / sec / 1e9,
                        "frac_of_measured_peak": nbytes / sec / 1e9 / peak, "frac_of_nominal_8000": nbytes / sec / 8e12})

    only = {t for t in args.only.split(",") if t}

    def want(group):
        return not only or group in only

    g = torch.Generator(device=dev).manual_seed(7)
    bf = torch.bfloat16
    # configs[2]: RMSNorm bf16 x[16,4096,4096], then out = silu(a) * b for a, b [65536, 11008]
    rows, D = 65536, 4096
    if want("rmsnorm") or want("addnorm"):
        _suite_norms(abi, timed, dev, g, rows, D, want)
    if want("gate"):
        _suite_gate(abi, timed, dev, g, rows)
    if want("embedding"):
        _suite_embedding(abi, timed, dev, g)
    if want("bert"):
        _suite_bert(abi, timed, dev, g)
    if want("rope"):
        _suite_rope(abi, timed, dev, g)
    if want("act"):
        _suite_act(abi, timed, dev, g)
    if want("attention"):
        _suite_attention(abi, timed, dev, g)
    if want("linear") and abi.linear_available():
        _suite_linear(abi, results, dev, g)
    abi.device_status()
    _emit({"suite": results, "peak_gbs": peak, "unit": "GB/s", "data": "synthetic",
           "note": "timings include torch's output allocation from its caching allocator"})


def _suite_norms(abi, timed, dev, g, rows, D, want):
    bf = torch.bfloat16
    x = torch.randn(rows, D, device=dev, generator=g).to(bf); dy = torch.randn(rows, D, device=dev, generator=g).to(bf)
    w = (1 + 0.02 * torch.randn(D, device=dev, generator=g)).to(bf)
    y, rstd = abi.rmsnorm_fwd(x, w, 1e-6)
    timed("rmsnorm_fwd bf16 [65536,4096]", lambda: abi.rmsnorm_fwd(x, w, 1e-6), 2 * rows * D * 2 + 4 * rows)
    timed("rmsnorm_bwd+reduce bf16 [65536,4096]", lambda: abi.rmsnorm_bwd(x, dy, w, rstd), 3 * rows * D * 2 + 4 * rows)
    # residual add + RMSNorm at the same shape (mamba.hpp:409-415), against add + norm as two passes
    r = torch.randn(rows, D, device=dev, generator=g).to(bf)
    sm_, yy, _, rs2 = abi.add_norm_fwd("rms", x, r, w, None, 1e-6)
    timed("add+rmsnorm_fwd bf16 [65536,4096] (2 reads, 2 writes)", lambda: abi.add_norm_fwd("rms", x, r, w, None, 1e-6),
          4 * rows * D * 2 + 4 * rows)
    timed("add+rmsnorm_bwd+reduce bf16 [65536,4096] (3 reads, 1 write)", lambda: abi.add_norm_bwd("rms", sm_, dy, r, w, None, rs2),
          4 * rows * D * 2 + 4 * rows)
    del x, dy, y, r, sm_, yy
    xf32 = torch.randn(32768, 1024, device=dev, generator=g); rf32 = torch.randn(32768, 1024, device=dev, generator=g)
    gf = torch.ones(1024, device=dev); bf_ = torch.zeros(1024, device=dev)
    s32, y32, m32, r32 = abi.add_norm_fwd("ln", xf32, rf32, gf, bf_, 1e-5)
    timed("add+layernorm_fwd fp32 [32768,1024]", lambda: abi.add_norm_fwd("ln", xf32, rf32, gf, bf_, 1e-5), 4 * 32768 * 1024 * 4)
    timed("add+layernorm_bwd+reduce fp32 [32768,1024]", lambda: abi.add_norm_bwd("ln", s32, xf32, rf32, gf, m32, r32), 4 * 32768 * 1024 * 4)
    del xf32, rf32, s32, y32


def _suite_gate(abi, timed, dev, g, rows):
    bf = torch.bfloat16
    H = 11008
    a = torch.randn(rows, H, device=dev, generator=g).to(bf); b = torch.randn(rows, H, device=dev, generator=g).to(bf)
    d = torch.randn(rows, H, device=dev, generator=g).to(bf)
    timed("silu_gate_fwd bf16 [65536,11008]", lambda: abi.silu_gate_fwd(a, b), 3 * rows * H * 2, iters=10)
    da, db = torch.empty_like(a), torch.empty_like(a)
    timed("silu_gate_bwd bf16 [65536,11008]", lambda: abi.silu_gate_bwd(a, b, d, da, db), 5 * rows * H * 2, iters=10)
    ab = torch.cat([a[:16384], b[:16384]], dim=1)              # SwiGLU form: halves of one [rows, 2H] tensor
    timed("silu_gate_fwd bf16 swiglu-strided [16384,2x11008]", lambda: abi.silu_gate_fwd(ab[:, :H], ab[:, H:]), 3 * 16384 * H * 2)
    del a, b, d, da, db, ab


def _suite_embedding(abi, timed, dev, g):
    bf = torch.bfloat16
    # configs[3]: gather table[32000,4096] bf16, ids int32 [32,2048]; rotary q,k [32,2048,32,128] bf16
    table = (0.02 * torch.randn(32000, 4096, device=dev, generator=g)).to(bf)
    ids = torch.randint(0, 32000, (32, 2048), device=dev, generator=g, dtype=torch.int32)
    timed("embedding_fwd bf16 65536 tokens x 4096", lambda: abi.embedding_fwd(table, ids), 2 * 65536 * 4096 * 2 + 65536 * 4)
    dout = torch.randn(65536, 4096, device=dev, generator=g).to(bf)
    timed("embedding_bwd bf16 (zero table + sort + segmented sum)", lambda: abi.embedding_bwd(dout, ids, 32000),
          65536 * 4096 * 2 + 32000 * 4096 * 2 + 65536 * 4, iters=10)
    index = abi.embedding_index(ids, 32000)
    timed("embedding_index int32 65536 ids (sort + row ranges; once per ids tensor, beside the forward gather)",
          lambda: abi.embedding_index(ids, 32000), 65536 * 4, iters=10)
    timed("embedding_bwd_indexed bf16 (segmented sum from a prebuilt index)", lambda: abi.embedding_bwd_indexed(dout, index, 32000),
          65536 * 4096 * 2 + 32000 * 4096 * 2, iters=10)
    del table, dout


def _suite_bert(abi, timed, dev, g):
    bf = torch.bfloat16
    # BERT front end (bert.hpp:155-194): vocab 30522, D 768, ids [256, 512]
    Bb, Sb, Db = 256, 512, 768
    wordt = (0.02 * torch.randn(30522, Db, device=dev, generator=g)).to(bf)
    post = (0.02 * torch.randn(512, Db, device=dev, generator=g)).to(bf); typt = (0.02 * torch.randn(2, Db, device=dev, generator=g)).to(bf)
    gb, bb = torch.ones(Db, device=dev).to(bf), torch.zeros(Db, device=dev).to(bf)
    idb = torch.randint(0, 30522, (Bb, Sb), device=dev, generator=g)
    yb, sb, mb, rb = abi.bert_embedding_ln_fwd(wordt, post, typt, idb, gb, bb)
    timed("bert_embedding+layernorm_fwd bf16 [256,512,768] (training: also writes the sum)",
          lambda: abi.bert_embedding_ln_fwd(wordt, post, typt, idb, gb, bb), 3 * Bb * Sb * Db * 2 + Bb * Sb * 8)
    timed("bert_embedding+layernorm_fwd bf16 [256,512,768] (inference)",
          lambda: abi.bert_embedding_ln_fwd(wordt, post, typt, idb, gb, bb, want_backward=False), 2 * Bb * Sb * Db * 2 + Bb * Sb * 8)
    timed("bert_embedding+layernorm_bwd bf16 (LN bwd + 3 table gradients)",
          lambda: abi.bert_embedding_ln_bwd(sb, yb, idb, gb, mb, rb, 30522, pos_rows=512), 4 * Bb * Sb * Db * 2 + 30522 * Db * 2, iters=10)
    del wordt, yb, sb


def _suite_rope(abi, timed, dev, g):
    bf = torch.bfloat16
    q = torch.randn(32, 2048, 32, 128, device=dev, generator=g).to(bf)
    cs = abi.rope_table(2048, 128)
    timed("rope_apply bf16 [32,2048,32,128] (one of q, k)", lambda: abi.rope_apply(q, cs), 2 * q.numel() * 2)
    timed("rope_apply inverse (backward)", lambda: abi.rope_apply(q, cs, inverse=True), 2 * q.numel() * 2)
    del q


def _suite_act(abi, timed, dev, g):
    n = 32 * 1024 * 1024
    xf = torch.randn(n, device=dev, generator=g); df = torch.randn(n, device=dev, generator=g)
    for nm, code in (("gelu", abi.ACT_GELU), ("silu", abi.ACT_SILU)):
        timed(f"{nm}_fwd fp32 32Mi", lambda: abi.act_fwd(xf, code), 2 * n * 4)
        timed(f"{nm}_bwd fp32 32Mi", lambda: abi.act_bwd(xf, df, code), 3 * n * 4)
    del xf, df


def _suite_attention(abi, timed, dev, g):
    bf = torch.bfloat16
    # attention probabilities (kernel.hpp:33-93): scores [16, 16, 1024, 1024], causal, then with an additive [B,T,S] mask
    for dt, nm in ((torch.float32, "fp32"), (bf, "bf16")):
        sc = torch.randn(16, 16, 1024, 1024, device=dev, generator=g).to(dt)
        da_ = torch.randn(16, 16, 1024, 1024, device=dev, generator=g).to(dt)
        at = abi.attention_softmax_fwd(sc, 0.125, causal=True)
        e = sc.element_size()
        timed(f"attention_softmax_fwd {nm} [16,16,1024,1024] causal", lambda: abi.attention_softmax_fwd(sc, 0.125, causal=True), 2 * sc.numel() * e)
        mk = torch.randn(16, 1024, 1024, device=dev, generator=g).to(dt)
        timed(f"attention_softmax_fwd {nm} [16,16,1024,1024] + mask [16,1024,1024]",
              lambda: abi.attention_softmax_fwd(sc, 0.125, attn_mask=mk), 2 * sc.numel() * e + mk.numel() * e)
        timed(f"attention_softmax_bwd {nm} [16,16,1024,1024]", lambda: abi.attention_softmax_bwd(at, da_, 0.125), 3 * sc.numel() * e)
        # with the dropout that follows (kernel.hpp:94): noise read in the same pass; training also writes the probabilities
        nz = ((torch.rand(16, 16, 1024, 1024, device=dev, generator=g) >= 0.1).float() / 0.9).to(dt)
        timed(f"attention_softmax+dropout_fwd {nm} [16,16,1024,1024] causal (2 reads, 2 writes)",
              lambda: abi.attention_softmax_fwd(sc, 0.125, causal=True, noise=nz), 4 * sc.numel() * e)
        timed(f"attention_softmax+dropout_bwd {nm} [16,16,1024,1024] (3 reads, 1 write)",
              lambda: abi.attention_softmax_bwd(at, da_, 0.125, noise=nz), 4 * sc.numel() * e)
        del sc, da_, at, mk, nz


def _suite_linear(abi, results, dev, g):
    """The FC layer with bias + GELU in the GEMM's epilogue (tensor cores, bf16) at feed-forward sizes, against the
    measured cuBLAS bf16 rate of this box and against libtorch's own linear -> gelu on the same tensors."""
    import torch.nn.functional as F
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peak_tf = float(json.loads(peaks_file.read_text())["bf16_tflops"]) if peaks_file.exists() else 1590.0
    bf = torch.bfloat16
    for (M, N, K) in ((16384, 4096, 1024), (16384, 1024, 4096), (32768, 3072, 768), (8192, 8192, 8192)):
        x = torch.randn(M, K, device=dev, generator=g).to(bf); w = (torch.randn(N, K, device=dev, generator=g) / K ** 0.5).to(bf)
        b = (0.1 * torch.randn(N, device=dev, generator=g)).to(bf)

        def timeit(fn, iters=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters / 1e3

        ours = timeit(lambda: abi.linear_bias_act_fwd(x, w, b, abi.ACT_GELU))
        ours_z = timeit(lambda: abi.linear_bias_act_fwd(x, w, b, abi.ACT_GELU, want_z=True))
        lib_ = timeit(lambda: F.gelu(F.linear(x, w, b)))
        flops = 2.0 * M * N * K
        results.append({"op": f"linear+bias+gelu bf16 [{M},{K}]x[{N},{K}]^T (tcgen05, epilogue fused)", "us": ours * 1e6,
                        "tflops": flops / ours / 1e12, "frac_of_measured_bf16_peak": flops / ours / 1e12 / peak_tf,
                        "with_pre_activation_output_us": ours_z * 1e6,
                        "libtorch_linear_then_gelu_us": lib_ * 1e6, "speedup_vs_libtorch": lib_ / ours,
                        "algorithmic_bytes": 2 * (M * K + N * K + M * N), "achieved_gbs": 2 * (M * K + N * K + M * N) / ours / 1e9,
                        "frac_of_measured_peak": None, "frac_of_nominal_8000": None})
        del x, w, b


# ------------------------------------------------------------ cfg5 sweep
def run_sweep(args, rank, world, local):
    """`--sweep`: the whole-box sweep configuration in one go: LayerNorm->GELU and RMSNorm->SiLU, fp32 and bf16,
    D in {768, 1024, 2048, 4096, 8192}, 2^20 rows split evenly over the ranks (strong scaling),
    forward / backward (+ partial reduce and, for N > 1, the sum over ranks) timed separately with CUDA
    events, max over ranks, with libtorch's CUDA ops on the same tensors beside them.  One JSON line."""
    import ctypes
    import torch.distributed as dist
    from thot_b200 import abi

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        box = [abi.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        comm = abi.Comm(box[0], rank, world, abi.EXCHANGE_PEER if args.exchange == "peer" else abi.EXCHANGE_NCCL, max_cols=2 * 8192)
    peak, _ = _peak()
    total_rows = 1 << 20
    iters = max(3, min(args.steps, 10))
    stream = torch.cuda.current_stream()
    st = ctypes.c_void_p(stream.cuda_stream)
    only = {t for t in args.only.split(",") if t}
    out = []
    for kind in ("ln", "rms"):
        for name in ("fp32", "bf16"):
            for D in (768, 1024, 2048, 4096, 8192):
                spec = f"cfg5:{kind}:{name}:{D}"
                if only and spec not in only and f"{kind}:{name}" not in only:
                    continue
                w = Workload(spec, world)
                r = StepRunner(w, comm, dev, seed=rank)
                rows = r.rows

                def f():
                    r.fwd(st)

                def bw():
                    r.bwd(st)
                    if comm is None:
                        r.reduce(st)
                    else:
                        comm.exchange_begin(r.partials, r.nparts.value, r.grads[0])
                        comm.exchange_end()

                res = {}
                for tag, fn, nbytes in (("fwd", f, 2 * rows * D * w.elt), ("bwd", bw, 3 * rows * D * w.elt)):
                    for _ in range(3):
                        fn()
                    if world > 1:
                        dist.barrier()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(iters):
                        fn()
                    e1.record()
                    torch.cuda.synchronize()
                    ms = e0.elapsed_time(e1) / iters
                    if world > 1:
                        t = torch.tensor([ms], device=dev)
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                        ms = float(t.item())
                    res[tag] = {"ms": ms, "gbs": nbytes * world / ms / 1e6, "frac_of_measured_per_gpu": nbytes / ms / 1e6 / peak,
                                "frac_of_nominal_8000_per_gpu": nbytes / ms / 1e6 / 8000.0}
                row = {"op": "LayerNorm->GELU" if kind == "ln" else "RMSNorm->SiLU", "dtype": name, "D": D,
                       "rows_total": total_rows, "rows_per_s_fwd_bwd": total_rows / ((res["fwd"]["ms"] + res["bwd"]["ms"]) / 1e3),
                       **{f"{k}_{m}": v[m] for k, v in res.items() for m in v}}
                if not args.no_comparator:
                    try:
                        cmpr = gpu_comparator(w, r, iters)
                        ours_same_rows = (res["fwd"]["ms"] + res["bwd"]["ms"]) * cmpr["rows"] / rows
                        row["gpu_comparator"] = {"rows": cmpr["rows"], "ms_per_step": cmpr["ms_per_step"],
                                                 "speedup": cmpr["ms_per_step"] / ours_same_rows}
                    except Exception as exc:
                        row["gpu_comparator"] = {"error": str(exc)}
                out.append(row)
                r.close()
                del r
                torch.cuda.empty_cache()
    abi.device_status()
    if rank == 0:
        _emit({"sweep": out, "n_gpus": world, "peak_gbs": peak, "scaling": "strong", "data": "synthetic",
               "exchange": "none" if world == 1 else args.exchange,
               "note": "backward includes the partial reduce and, for N > 1, the sum over ranks; gpu_comparator = libtorch CUDA ops "
                       "(forward + autograd backward) on a bounded row sample of the same tensors"})
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------ our arm
def _emit(line: dict) -> None:
    """The one JSON line goes to the process's original stdout; everything else that libraries
    print to fd 1 (NCCL's version banner, for one) was redirected to stderr in main()."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = 1


def _peak():
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        return float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback"


class StepRunner:
    """One workload on this rank: device-resident synthetic inputs, the C step driver
    (nb2_step_run: forward, end of the previous exchange, backward, partial reduce + exchange),
    and the same kernels one by one for the per-kernel timings."""

    def __init__(self, w: Workload, comm, dev, seed: int):
        import ctypes
        from thot_b200 import abi

        self.abi, self.w, self.comm, self.dev = abi, w, comm, dev
        rows, D = w.rows_per_rank, w.D
        self.rows, self.D = rows, D
        self.x, self.dy, self.gamma, self.beta = synth_inputs(w, rows, dev, seed)
        self.code = abi.dtype_code(w.dtype)
        self.y, self.dx = torch.empty_like(self.x), torch.empty_like(self.x)
        self.ncols = (2 if w.kind == "ln" else 1) * D
        self.grads = [torch.zeros(self.ncols, dtype=torch.float32, device=dev) for _ in range(2)]
        self.step = abi.NormStep(comm, w.kind, rows, D, w.dtype, w.act, w.eps)
        self.k = 0
        # buffers of the one-by-one launches
        self.mean = torch.empty(max(rows, 1), dtype=torch.float32, device=dev)
        self.rstd = torch.empty(max(rows, 1), dtype=torch.float32, device=dev)
        self.partials = torch.empty(abi.workspace_bytes(abi.WS_NORM_BWD, rows, D, self.code) // 4, dtype=torch.float32, device=dev)
        self.nparts = ctypes.c_int64(0)
        self._ct = ctypes

    def run(self):
        self.step.run(self.x, self.dy, self.gamma, self.beta, self.y, self.dx, self.grads[self.k & 1])
        self.k += 1

    def finish(self):
        self.step.finish()

    # ---- the same kernels, one launch each
    def _ptrs(self):
        P = lambda t: None if t is None else self._ct.c_void_p(t.data_ptr())  # noqa: E731
        return P

    def fwd(self, st):
        abi, w, P, L = self.abi, self.w, self._ptrs(), self.abi.lib()
        if w.kind == "ln":
            abi.check(L.nb2_layernorm_fwd(P(self.x), P(self.gamma), P(self.beta), P(self.y), P(self.mean), P(self.rstd),
                                          self.rows, self.D, w.eps, self.code, w.act, st))
        else:
            abi.check(L.nb2_rmsnorm_fwd(P(self.x), P(self.gamma), P(self.y), P(self.rstd), self.rows, self.D, w.eps, self.code, w.act, st))

    def bwd(self, st):
        abi, w, P, L = self.abi, self.w, self._ptrs(), self.abi.lib()
        if w.kind == "ln":
            abi.check(L.nb2_layernorm_bwd(P(self.x), P(self.dy), P(self.gamma), P(self.beta), P(self.mean), P(self.rstd), P(self.dx),
                                          P(self.partials), self._ct.byref(self.nparts), self.rows, self.D, self.code, w.act, st))
        else:
            abi.check(L.nb2_rmsnorm_bwd(P(self.x), P(self.dy), P(self.gamma), P(self.rstd), P(self.dx), P(self.partials),
                                        self._ct.byref(self.nparts), self.rows, self.D, self.code, w.act, st))

    def reduce(self, st):
        """The partial reduce; with a communicator, the call that also starts (and, one call later, completes) the
        sum over ranks, as the step driver issues it."""
        abi, P, L = self.abi, self._ptrs(), self.abi.lib()
        if self.comm is None:
            abi.check(L.nb2_colreduce_partials(P(self.partials), self.nparts.value, self.ncols, P(self.grads[0]), st))
        else:
            self.k += 1
            abi.check(L.nb2_grad_exchange_begin(self.comm.handle, P(self.partials), self.nparts.value, self.ncols, P(self.grads[self.k & 1]), st))

    def close(self):
        self.step.close()


def make_comm(abi, dist, rank, world, mode, dev):
    """The library's communicator for this run.  Before any timing the exchange is checked once against
    torch.distributed on a known vector; if the peer form cannot be set up or does not agree on this box (no peer
    access between some pair of GPUs, say) every rank switches to the NCCL form together and the JSON line says so."""
    def build(m):
        box = [abi.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return abi.Comm(box[0], rank, world, m, max_cols=2 * 8192)

    def agrees(c):
        v = torch.arange(4096, device=dev, dtype=torch.float32) * (rank + 1) * 0.25
        want = v.clone()
        dist.all_reduce(want)
        for _ in range(3):                                   # both slot parities
            got = v.clone()
            c.allreduce_(got)
        torch.cuda.synchronize()
        abi.device_status()
        return bool(torch.equal(got, want))

    note = None
    ok, comm = 1, None
    try:
        comm = build(mode)
        ok = 1 if agrees(comm) else 0
    except Exception as exc:                                 # set-up or a bounded wait that ran out
        ok, note = 0, str(exc)[:200]
    flag = torch.tensor([ok], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 1:
        return comm, mode, None
    if mode == abi.EXCHANGE_NCCL:
        raise SystemExit(f"bench: the gradient exchange does not work on this box ({note})")
    try:
        if comm is not None:
            comm.close()
    except Exception:
        pass
    comm = build(abi.EXCHANGE_NCCL)
    if not agrees(comm):
        raise SystemExit("bench: neither exchange form works on this box")
    return comm, abi.EXCHANGE_NCCL, "peer form failed its self-check on this box (%s); NCCL form used" % (note or "result mismatch")


def timed_steps(runner: StepRunner, steps: int, warmup: int, world: int, dev, clocks=None, trace=None):
    """W untimed steps, then exactly K steps between barrier + synchronize on both sides, CUDA events
    on the launching stream, max over ranks.  Returns seconds per step.  `trace` (a dict) receives this
    rank's per-step series: device time between consecutive steps' events and host time per launch call."""
    import torch.distributed as dist

    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        runner.run()
    runner.finish()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clocks is not None:
        clocks.armed = True
    step_ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps)] if trace is not None else None
    host_t = []
    e0.record(stream)
    for i in range(steps):
        if trace is not None:
            t0 = time.perf_counter()
        runner.run()
        if trace is not None:
            step_ev[i].record(stream)
            host_t.append((time.perf_counter() - t0) * 1e6)
    runner.finish()                              # the last exchange is inside the timed region
    e1.record(stream)
    if clocks is not None:
        clocks.sample()                          # the queue is still draining here
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.armed = False
    ms = e0.elapsed_time(e1)
    if trace is not None:
        marks = [e0] + step_ev
        trace["device_us_per_step"] = [round(marks[i].elapsed_time(marks[i + 1]) * 1e3, 1) for i in range(steps)]
        trace["host_us_per_launch"] = [round(v, 1) for v in host_t]
        trace["rank_ms"] = ms
    barrier()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / 1e3 / steps


def kernel_times(runner: StepRunner, n_prof: int):
    """Per-kernel durations inside a step sequence: CUDA events around each launch."""
    import ctypes
    stream = torch.cuda.current_stream()
    st = ctypes.c_void_p(stream.cuda_stream)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_prof)]
    for i in range(3):
        runner.fwd(st); runner.bwd(st); runner.reduce(st)
    runner.finish()
    torch.cuda.synchronize()
    for i in range(n_prof):
        ev[i][0].record(stream); runner.fwd(st)
        ev[i][1].record(stream); runner.bwd(st)
        ev[i][2].record(stream); runner.reduce(st)
        ev[i][3].record(stream)
    runner.finish()
    torch.cuda.synchronize()
    t_fwd = float(np.mean([ev[i][0].elapsed_time(ev[i][1]) for i in range(n_prof)])) / 1e3
    t_bwd = float(np.mean([ev[i][1].elapsed_time(ev[i][2]) for i in range(n_prof)])) / 1e3
    t_red = float(np.mean([ev[i][2].elapsed_time(ev[i][3]) for i in range(n_prof)])) / 1e3
    return t_fwd, t_bwd, t_red


def gpu_comparator(w: Workload, runner: StepRunner, steps: int):
    """What the reference executes when its tensors live on a GPU: libtorch's CUDA ops, unfused.
    LayerNorm: layer_norm -> gelu(erf) (classic.hpp:436,451); RMSNorm: the op chain of
    mamba.hpp:134-140 (pow, mean, +eps, rsqrt, mul, mul) -> silu; forward + autograd backward with the
    same dY on the same device tensors, CUDA-event timed.  Rows are bounded so that autograd's saved
    tensors fit beside the benchmark's own buffers."""
    import torch.nn.functional as F

    rows = min(runner.rows, (1 << 30) // max(w.D * w.elt // 2, 1))      # at most ~2 GiB per tensor
    if rows <= 0:
        return None
    x = runner.x[:rows].detach().requires_grad_(True)
    dy = runner.dy[:rows]
    g = runner.gamma.detach().requires_grad_(True)
    b = runner.beta.detach().requires_grad_(True) if runner.beta is not None else None

    def one():
        if w.kind == "ln":
            y = F.gelu(F.layer_norm(x, (w.D,), g, b, w.eps))
        else:
            variance = x.pow(2).mean(-1, True)
            y = F.silu(x * torch.rsqrt(variance + w.eps) * g)
        y.backward(dy)
        x.grad = None
        g.grad = None
        if b is not None:
            b.grad = None

    n = max(3, min(steps, 10))
    for _ in range(3):
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        one()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / n
    del x, g, b
    torch.cuda.empty_cache()
    return {"what": "libtorch CUDA " + ("layer_norm -> gelu(erf)" if w.kind == "ln" else "pow/mean/rsqrt/mul/mul -> silu") + ", forward + autograd backward",
            "rows": rows, "steps": n, "ms_per_step": sec * 1e3, "value": w.step_bytes(rows) / sec / 1e9, "unit": UNIT,
            "rows_per_s": rows / sec}


def e2e_run(w: Workload, runner: StepRunner, steps: int, world: int, dev):
    """The same metric through the host-buffer C-ABI call: pinned host tensors in and out, the
    host<->device copies inside the timed region.  PCIe-bound by construction."""
    import torch.distributed as dist
    abi = runner.abi
    D = w.D
    e2e_rows = min(runner.rows, (512 << 20) // (D * w.elt))       # pinned host buffers of at most 512 MiB each
    if e2e_rows <= 0:
        return None
    hs = abi.HostStep(e2e_rows, D, w.dtype)
    hx = runner.x[:e2e_rows].cpu().pin_memory(); hdy = runner.dy[:e2e_rows].cpu().pin_memory()
    hg = runner.gamma.cpu()
    hb = runner.beta.cpu() if runner.beta is not None else None
    hy = torch.empty_like(hx).pin_memory(); hdx = torch.empty_like(hx).pin_memory()
    hgr = torch.empty(runner.ncols, dtype=torch.float32).pin_memory()

    def one():
        if w.kind == "ln":
            hs.step(hx, hdy, hg, hb, hy, hdx, hgr, w.eps, w.act)
        else:
            hs.step_rms(hx, hdy, hg, hy, hdx, hgr, w.eps, w.act)

    n_e2e = max(3, min(steps, 30))
    for _ in range(3):
        one()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        one()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / n_e2e
    if world > 1:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    hs.close()
    act_bytes = e2e_rows * D * w.elt
    nparam = (2 if w.kind == "ln" else 1) * D
    return {"value": w.step_bytes(e2e_rows) * world / dt / 1e9, "unit": UNIT,
            "h2d_bytes_per_step": 2 * act_bytes + nparam * w.elt, "d2h_bytes_per_step": 2 * act_bytes + nparam * 4,
            "ms_per_step": dt * 1e3, "rows_per_step": e2e_rows, "steps": n_e2e,
            "call": ("nb2_layernorm_act_step_host" if w.kind == "ln" else "nb2_rmsnorm_act_step_host")
                    + " (x, dY in pinned host memory; y, dX, parameter gradients out)",
            "note": "bound by the host link: every step moves 4 activation tensors over PCIe, the kernels are idle most of the time"}


def main():
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="how the parameter gradients are summed over ranks: the library's own peer-store exchange fused into "
                         "the partial reduce (default: measured faster at 2 and 4 GPUs, no SM held by a collective), or an NCCL "
                         "allreduce on a side stream")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-comparator", action="store_true")
    ap.add_argument("--no-cfg2", action="store_true", help="skip the x[32,1024,1024] sub-record")
    ap.add_argument("--reserve-sms", type=int, default=0,
                    help="SMs the persistent norm kernels leave to a kernel that runs beside them (default 0)")
    ap.add_argument("--trace-steps", action="store_true",
                    help="record one CUDA event and one host timestamp per step and print every rank's series to stderr")
    ap.add_argument("--sweep", action="store_true", help="whole-box sweep: 2^20 rows x D in {768..8192}, both norms, both dtypes")
    ap.add_argument("--suite", action="store_true", help="time the other kernels of the path (1 GPU) instead of the step")
    ap.add_argument("--only", default="", help="with --suite: run only the groups named here, comma separated "
                    "(rmsnorm, addnorm, gate, embedding, bert, rope, act, attention, linear); with --sweep: only these points "
                    "(cfg5:ln:bf16:2048 or ln:bf16)")
    args = ap.parse_args()
    if args.warmup < 3:
        print(f"bench: --warmup {args.warmup} is below the 3 warm-up steps the timing rules ask for", file=sys.stderr)

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    w = Workload(args.workload, world)

    if args.impl == "reference":
        run_reference_arm(args, w, rank, world)
        return
    if args.suite:
        if rank == 0:
            run_suite(args)
        return
    if args.sweep:
        run_sweep(args, rank, world, local)
        return

    import torch.distributed as dist
    from thot_b200 import abi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    clocks = ClockSampler(local).start()          # before the warm-up; it samples only inside the timed region
    comm = None
    mode = abi.EXCHANGE_PEER if args.exchange == "peer" else abi.EXCHANGE_NCCL
    exchange_note = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)     # plumbing: barrier, max over ranks, passing the id
        comm, mode, exchange_note = make_comm(abi, dist, rank, world, mode, dev)
    abi.lib().nb2_reserve_sms(max(args.reserve_sms, 0))

    runner = StepRunner(w, comm, dev, seed=1234 + rank)
    trace = {} if args.trace_steps else None
    sec_per_step = timed_steps(runner, args.steps, args.warmup, world, dev, clocks, trace)
    clocks.stop()
    if trace is not None:
        print("STEP_TRACE " + json.dumps({"rank": rank, "workload": w.spec, **trace}), file=sys.stderr, flush=True)
    value = w.step_bytes() * world / sec_per_step / 1e9

    # ---- per-kernel durations inside the same step sequence (CUDA events around each launch)
    t_fwd, t_bwd, t_red = kernel_times(runner, min(args.steps, 50))
    peak, peak_src = _peak()
    traffic = None
    tf = ROOT / "profiles" / "traffic.json"
    if tf.exists():
        traffic = json.loads(tf.read_text()).get(f"{w.kind}_bwd:{w.spec}")
    bwd_gbs = w.bwd_bytes() / t_bwd / 1e9
    fwd_gbs = w.fwd_bytes() / t_fwd / 1e9
    roofline = {"bound": "hbm", "kernel": "norm_bwd_tma_kernel (dX + dgamma/dbeta partials)", "achieved": bwd_gbs,
                "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak, "traffic": traffic, "peak_source": peak_src,
                "frac_of_nominal_8000": bwd_gbs / 8000.0,
                "algorithmic_bytes_per_launch": w.bwd_bytes(), "launch_us": t_bwd * 1e6}
    kernels = {
        "norm_fwd_kernel": {"ms": t_fwd * 1e3, "achieved_gbs": fwd_gbs, "frac": fwd_gbs / peak, "frac_of_nominal_8000": fwd_gbs / 8000.0},
        "norm_bwd_kernel": {"ms": t_bwd * 1e3, "achieved_gbs": bwd_gbs, "frac": bwd_gbs / peak, "frac_of_nominal_8000": bwd_gbs / 8000.0},
        "colreduce_kernel": {"ms": t_red * 1e3},
    }

    comparator = None
    if not args.no_comparator:
        try:
            comparator = gpu_comparator(w, runner, args.steps)
            if comparator is not None:
                comparator["ours_ms_per_step_same_rows"] = sec_per_step * 1e3 * comparator["rows"] / max(runner.rows, 1)
                comparator["speedup"] = (value / world) / comparator["value"]
        except Exception as exc:
            comparator = {"error": str(exc)}

    e2e = None
    if not args.no_e2e:
        e2e = e2e_run(w, runner, args.steps, world, dev)

    # ---- x[32,1024,1024] per GPU as a sub-record: a 0.12 ms step, where fixed per-step costs show
    cfg2 = None
    if not args.no_cfg2 and w.spec != "cfg2":
        w2 = Workload("cfg2", world)
        r2 = StepRunner(w2, comm, dev, seed=4321 + rank)
        trace2 = {} if args.trace_steps else None
        s2 = timed_steps(r2, max(args.steps, 200), max(args.warmup, 10), world, dev, None, trace2)
        if trace2 is not None:
            print("STEP_TRACE " + json.dumps({"rank": rank, "workload": "cfg2", **trace2}), file=sys.stderr, flush=True)
        f2, b2, c2 = kernel_times(r2, 50)
        cfg2 = {"workload": w2.name, "scaling": "weak", "ms_per_step": s2 * 1e3, "value": w2.step_bytes() * world / s2 / 1e9, "unit": UNIT,
                "rows_per_s": w2.rows_per_rank * world / s2, "steps": max(args.steps, 200),
                "fwd": {"ms": f2 * 1e3, "frac": w2.fwd_bytes() / f2 / 1e9 / peak, "frac_of_nominal_8000": w2.fwd_bytes() / f2 / 8e12},
                "bwd": {"ms": b2 * 1e3, "frac": w2.bwd_bytes() / b2 / 1e9 / peak, "frac_of_nominal_8000": w2.bwd_bytes() / b2 / 8e12},
                "colreduce_ms": c2 * 1e3}
        if not args.no_comparator:
            try:
                cmp2 = gpu_comparator(w2, r2, 10)
                cfg2["gpu_comparator"] = {"ms_per_step": cmp2["ms_per_step"], "speedup": (cfg2["value"] / world) / cmp2["value"]}
            except Exception as exc:
                cfg2["gpu_comparator"] = {"error": str(exc)}
        r2.close()
        del r2

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu = reference_cpu_run(w, 1000, 2, budget_s=15.0)[4]
        except Exception as exc:      # a missing oracle must not hide the GPU numbers
            cpu = {"error": str(exc)}

    status = abi.device_status()
    launches_per_step = 3          # forward, backward, partial reduce (+ exchange in the same kernel in the peer form)
    if rank == 0:
        if world == 1:
            exchange = "none"
        elif mode == abi.EXCHANGE_NCCL:
            exchange = ("ncclAllReduce of [%d] fp32 per step, issued by the C step driver on the communicator's side stream; "
                        "it overlaps the next step's forward" % runner.ncols)
        else:
            exchange = ("peer-store exchange of [%d] fp32 per step: the partial-reduce kernel stores this rank's sums into every "
                        "peer's buffer over NVLink and, one step later, adds the ranks' sums in rank order" % runner.ncols)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
            "scaling": w.scaling, "vs_baseline": None,
            "dtype": "f32" if w.dtype == torch.float32 else "bf16", "data": "synthetic",
            "config": config_of(w, world),
            "exchange": exchange, "exchange_note": exchange_note, "reserved_sms": max(args.reserve_sms, 0),
            "rows_per_s": w.rows_per_rank * world / sec_per_step,
            "frac_of_measured_per_gpu": value / world / peak,
            "frac_of_nominal_8000_per_gpu": value / world / 8000.0,
            "roofline": roofline, "kernels": kernels, "gpu_comparator": comparator, "cpu_baseline": cpu, "e2e": e2e,
            "cfg2": cfg2, "device_status": status,
            "clocks": clocks.summary(), "gpu_launches": launches_per_step * args.steps,
        }
        _emit(line)
    runner.close()
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
