"""Helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np
import torch

import triattention_oracle as orc

# FP tolerance of the parity contract: max-abs 2e-3 and cosine >= 0.9999 against the reference kernel.
# Outputs are bf16 (8 significant bits): two correct kernels can round the same value to neighbouring
# bf16 numbers, so comparisons of bf16 outputs add one bf16 ulp of the reference value,
# 2^(floor(log2|x|) - 7), to the absolute bound.  The mean absolute error is held to ABS_TOL / 4 so that
# the ulp allowance cannot hide a systematic error.
ABS_TOL, COS_TOL = 2e-3, 0.9999


def ulp_diff(a, b) -> np.ndarray:
    """Distance in float32 ulps (same sign assumed, which holds for scales)."""
    ia = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    ib = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    return np.abs(ia - ib)


def fp_report(got, ref, bf16_ulp=True, ulp_digits=7):
    """ulp_digits: explicit significand bits of the output type the two sides were rounded to (7 = bf16, 10 = fp16)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** -120))) - ulp_digits)
    tol = ABS_TOL + (ulp if bf16_ulp else 0.0)
    err = np.abs(got - ref)
    cos = float((got * ref).sum() / max(np.linalg.norm(got) * np.linalg.norm(ref), 1e-30))
    return dict(max_abs=float(err.max()), worst_excess=float((err - tol).max()), mean_abs=float(err.mean()), cos=cos)


def assert_fp_close(got, ref, what, bf16_ulp=True, ulp_digits=7):
    r = fp_report(got, ref, bf16_ulp, ulp_digits)
    assert r["worst_excess"] <= 0 and r["cos"] >= COS_TOL and r["mean_abs"] <= ABS_TOL / 4, f"{what}: {r}"
    return r


def bf16_cuda(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).cuda()


def from_bits(bits):
    """uint16 bf16 bit patterns -> float32."""
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def code_mismatch(got, ref):
    """(fraction of differing codes, largest absolute difference)."""
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    return float((d != 0).mean()), int(d.max())


def make_inputs(hq, hk, t, seed, batch=1, dims=(7, 42, 77, 113), scale=4.0, fraction=None):
    """[B,H,T,128] float32 arrays of bf16 values."""
    mk = lambda h, s: np.stack([orc.synth((h, t, 128), s + 1000 * b, outlier_dims=None if fraction else dims,
                                          outlier_scale=scale, outlier_fraction=fraction) for b in range(batch)])
    return mk(hq, seed), mk(hk, seed + 1), np.stack([orc.synth((hk, t, 128), seed + 2 + 1000 * b) for b in range(batch)])
