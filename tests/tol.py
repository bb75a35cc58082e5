"""Tolerances of the parity tests, in one place.

fp32 outputs  : |got - ref| <= 1e-6 + 1e-5 * |ref|
bf16 outputs  : within 2 bf16 ulp of the fp32-accumulated result rounded to bf16, or
    inside the fp32 absolute tolerance (1e-6): where fp32 arithmetic itself cancels
    (GELU's 1 + erf(z/sqrt2) for z < -5 is a multiple of 6e-8) a bf16 output cannot be
    held to a tighter absolute error than the fp32 path it is computed in.
fp32 outputs against the LIVE fp32 reference (libtorch CPU) are adjudicated by the fp64
    result where one exists: an element passes when inside the tolerance of the fp32
    reference OR at least as close to fp64 as the fp32 reference is.  (libtorch's fp32
    CPU GELU is itself 1.1e-6 off in the tail around z = -3.5.)
long fp32 sums over n rows (dgamma, dbeta, dweight), `long_sum_close`.  Each element is classified
    by the first rule it meets, and the call returns how many elements met which:
      tol64  : |got - ref64| <= 1e-6 + 1e-5 |ref64|, the stated tolerance against the exact (fp64) sum;
      tol32  : the stated tolerance against the fp32 CPU reference (libtorch through the reference's
               own modules), when one is given;
      closer : at least as close to the fp64 sum as the fp32 CPU reference is;
      vector : the element met none of the above (its fp32 CPU value happens to lie nearer the exact
               sum than ours), but over the whole vector the GPU result is closer to fp64 than the
               fp32 CPU reference in BOTH the largest and the root-mean-square distance;
      sqrt_n : |got - ref64| <= 1e-6 + 1e-5 max(|ref64|, sqrt(n)): a sum of n unit-scale terms has
               natural magnitude sqrt(n) even where it cancels to ~0, and any fp32 accumulation
               carries an error proportional to that.  This rule is NOT part of the stated
               tolerance.  It is accepted only where no fp32 CPU reference exists for the case
               (`strict=False`: small shape sweeps against the C oracle, consistency properties
               between two GPU results); with `strict=True` (every configuration-sized case) an
               element that only this rule admits fails the test.
integer / byte outputs: exact.
"""
from __future__ import annotations

import numpy as np

FP32_RTOL, FP32_ATOL = 1e-5, 1e-6
BF16_MAX_ULP = 2


def fp32_close(got, ref, rtol=FP32_RTOL, atol=FP32_ATOL):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = np.abs(got - ref)
    bound = atol + rtol * np.abs(ref)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{bad.sum()} of {bad.size} elements outside 1e-5 rel / 1e-6 abs; worst at {i}: "
                             f"got {got[i]!r} ref {ref[i]!r} err {err[i]:.3e}")


def fp32_close_adjudicated(got, ref32, ref64):
    """got vs the live fp32 reference, with the fp64 result as arbiter (see module docstring)."""
    got = np.asarray(got, np.float64); ref32 = np.asarray(ref32, np.float64); ref64 = np.asarray(ref64, np.float64)
    ok = np.abs(got - ref32) <= FP32_ATOL + FP32_RTOL * np.abs(ref32)
    slack = np.spacing(np.abs(ref64).astype(np.float32)).astype(np.float64)
    ok |= np.abs(got - ref64) <= np.abs(ref32 - ref64) + slack
    if not ok.all():
        i = np.unravel_index(np.argmax(~ok), ok.shape)
        raise AssertionError(f"{(~ok).sum()} of {ok.size} elements neither within tolerance of the fp32 reference nor "
                             f"closer to fp64; first at {i}: got {got[i]!r} ref32 {ref32[i]!r} ref64 {ref64[i]!r}")


PARITY_LOG = []          # one record per labelled long_sum_close call; written out by tests/conftest.py


def long_sum_close(got, ref64, n_terms, ref32=None, strict=False, label=None):
    """dgamma/dbeta/dweight over `n_terms` rows; see the module docstring for the rules.
    Returns {"tol64": k, "tol32": k, "closer": k, "vector": k, "sqrt_n": k, ...distances}."""
    got = np.asarray(got, np.float64).ravel(); ref64 = np.asarray(ref64, np.float64).ravel()
    assert got.shape == ref64.shape, (got.shape, ref64.shape)
    if strict and ref32 is None:
        raise ValueError("strict long-sum check needs the fp32 CPU reference")
    d_gpu = np.abs(got - ref64)
    rule = np.full(got.shape, "", dtype=object)
    rule[d_gpu <= FP32_ATOL + FP32_RTOL * np.abs(ref64)] = "tol64"
    stats = {"n_terms": int(n_terms), "elements": int(got.size), "max_dist_gpu_to_f64": float(d_gpu.max(initial=0.0)),
             "rms_dist_gpu_to_f64": float(np.sqrt(np.mean(d_gpu ** 2))) if got.size else 0.0}
    if ref32 is not None:
        ref32 = np.asarray(ref32, np.float64).ravel()
        d_ref = np.abs(ref32 - ref64)
        slack = np.spacing(np.abs(ref64).astype(np.float32)).astype(np.float64)
        rule[(rule == "") & (np.abs(got - ref32) <= FP32_ATOL + FP32_RTOL * np.abs(ref32))] = "tol32"
        rule[(rule == "") & (d_gpu <= d_ref + slack)] = "closer"
        stats.update(max_dist_f32cpu_to_f64=float(d_ref.max(initial=0.0)), rms_dist_f32cpu_to_f64=float(np.sqrt(np.mean(d_ref ** 2))))
        if stats["max_dist_gpu_to_f64"] <= stats["max_dist_f32cpu_to_f64"] and stats["rms_dist_gpu_to_f64"] <= stats["rms_dist_f32cpu_to_f64"]:
            rule[rule == ""] = "vector"
    scale = np.maximum(np.abs(ref64), float(n_terms) ** 0.5)
    rule[(rule == "") & (d_gpu <= FP32_ATOL + FP32_RTOL * scale)] = "sqrt_n"
    counts = {k: int((rule == k).sum()) for k in ("tol64", "tol32", "closer", "vector", "sqrt_n")}
    stats.update(counts)
    if label is not None:
        PARITY_LOG.append(dict(stats, label=label, strict=bool(strict)))
    bad = rule == ""
    if strict:
        bad |= rule == "sqrt_n"
    if bad.any():
        i = int(np.argmax(bad))
        r32 = ref32[i] if ref32 is not None else float("nan")
        raise AssertionError(f"{int(bad.sum())} of {bad.size} long sums fail ({'strict' if strict else 'lenient'}; rules met: {counts}); "
                             f"first at {i}: got {got[i]!r} ref32 {r32!r} ref64 {ref64[i]!r}")
    return stats


def to_bf16_bits(a) -> np.ndarray:
    """Round fp32/fp64 values to bf16 (nearest even) and return the 16-bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def _ordered(bits):
    b = np.asarray(bits, np.uint16).astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)


def bf16_ulp_mask(got_bits, ref_values, max_ulp=BF16_MAX_ULP):
    """Elementwise pass mask of the bf16 rule (2 ulp, or inside the fp32 absolute tolerance)."""
    d = np.abs(_ordered(got_bits) - _ordered(to_bf16_bits(ref_values)))
    inside_abs = np.abs(bf16_bits_to_f32(got_bits).astype(np.float64) - np.asarray(ref_values, np.float64)) <= FP32_ATOL
    return (d <= max_ulp) | inside_abs


def bf16_ulp_close(got_bits, ref_values, max_ulp=BF16_MAX_ULP):
    """got_bits: uint16 bf16 patterns; ref_values: fp32/fp64 reference before rounding."""
    ref_bits = to_bf16_bits(ref_values)
    d = np.abs(_ordered(got_bits) - _ordered(ref_bits))
    inside_abs = np.abs(bf16_bits_to_f32(got_bits).astype(np.float64) - np.asarray(ref_values, np.float64)) <= FP32_ATOL
    d = np.where(inside_abs, 0, d)
    if (d > max_ulp).any():
        i = np.unravel_index(np.argmax(d), d.shape)
        raise AssertionError(f"{(d > max_ulp).sum()} of {d.size} elements differ by more than {max_ulp} bf16 ulp; "
                             f"worst {d[i]} ulp at {i}: got {bf16_bits_to_f32(got_bits)[i]!r} ref {np.asarray(ref_values)[i]!r}")
