"""Comparison helpers shared by the parity tests."""
import numpy as np

# North-star tolerances: max-abs error relative to the reference tensor's max-abs.
TOL_F32 = 1e-4
TOL_F16 = 2e-2
# The reference's own absolute tolerances (tests/gpt.rs:8-9): CPU 1e-4, accelerators 2e-3.
REF_ABS_TOL_ACCEL = 2e-3


def rel_err(got, want) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "non-finite values in result"
    denom = max(np.abs(want).max(), 1e-30)
    return float(np.abs(got - want).max() / denom)


def assert_close(got, want, tol, label):
    e = rel_err(got, want)
    assert e <= tol, f"{label}: max-abs rel error {e:.3e} > {tol:.1e}"
    return e
