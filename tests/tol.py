"""Tolerances of the parity tests, in one place.

fp32 outputs  : |got - ref| <= 1e-6 + 1e-5 * |ref|
bf16 outputs  : within 2 bf16 ulp of the fp32-accumulated result rounded to bf16
long fp32 sums (dgamma, dbeta, dweight): the fp32 tolerance against the fp32
    reference, OR at least as close to the fp64 result as the fp32 reference is
    (a different summation order of 1e4..1e6 terms is not an error).
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


def long_sum_close(got, ref32, ref64, scale_atol=None):
    """dgamma/dbeta/dweight: pass per element if inside the fp32 tolerance of the fp32
    reference or not farther from the fp64 reference than the fp32 reference is
    (plus one fp32 ulp of slack)."""
    got = np.asarray(got, np.float64); ref32 = np.asarray(ref32, np.float64); ref64 = np.asarray(ref64, np.float64)
    ok_tol = np.abs(got - ref32) <= FP32_ATOL + FP32_RTOL * np.abs(ref32)
    slack = np.spacing(np.abs(ref64).astype(np.float32)).astype(np.float64)
    ok_f64 = np.abs(got - ref64) <= np.abs(ref32 - ref64) + slack
    ok_abs = np.abs(got - ref64) <= FP32_ATOL + FP32_RTOL * np.abs(ref64)
    bad = ~(ok_tol | ok_f64 | ok_abs)
    if bad.any():
        i = int(np.argmax(bad))
        raise AssertionError(f"{bad.sum()} of {bad.size} long sums fail; first at {i}: got {got.flat[i]!r} "
                             f"ref32 {ref32.flat[i]!r} ref64 {ref64.flat[i]!r}")


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


def bf16_ulp_close(got_bits, ref_values, max_ulp=BF16_MAX_ULP):
    """got_bits: uint16 bf16 patterns; ref_values: fp32/fp64 reference before rounding."""
    ref_bits = to_bf16_bits(ref_values)
    d = np.abs(_ordered(got_bits) - _ordered(ref_bits))
    if (d > max_ulp).any():
        i = np.unravel_index(np.argmax(d), d.shape)
        raise AssertionError(f"{(d > max_ulp).sum()} of {d.size} elements differ by more than {max_ulp} bf16 ulp; "
                             f"worst {d[i]} ulp at {i}: got {bf16_bits_to_f32(got_bits)[i]!r} ref {np.asarray(ref_values)[i]!r}")
