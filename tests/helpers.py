"""Shared helpers of the parity tests: seeded inputs and the reference's comparison rule."""
from __future__ import annotations

import numpy as np


def assert_all_close(name, actual, expected, tol):
    """Port of the reference's `assert_all_close` (crates/cleandl/tests/common/mod.rs:240-280):
    fails on any NaN or any |actual - expected| > tol, reporting the worst offenders."""
    actual = np.asarray(actual, dtype=np.float64).ravel()
    expected = np.asarray(expected, dtype=np.float64).ravel()
    tol = np.broadcast_to(np.asarray(tol, dtype=np.float64).ravel(), expected.shape) \
        if np.ndim(tol) else np.full(expected.shape, float(tol))
    assert actual.shape == expected.shape, f"{name}: shape {actual.shape} vs {expected.shape}"
    err = np.abs(actual - expected)
    bad = ~(err <= tol)  # NaN compares false, so NaN is bad
    if bad.any():
        idx = np.argsort(-(np.where(np.isnan(err), np.inf, err) / np.maximum(tol, 1e-30)))[:8]
        lines = [f"  [{i}] got {actual[i]:.6g} expected {expected[i]:.6g} tol {tol[i]:.3g}" for i in idx]
        raise AssertionError(f"{name}: {int(bad.sum())} of {bad.size} elements out of tolerance\n"
                             + "\n".join(lines))


def to_f32(t):
    """torch tensor (any dtype/device) -> float32 numpy."""
    return t.detach().float().cpu().numpy()
