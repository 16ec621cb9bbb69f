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


# A tensor that is exactly zero in the reference (dQ at T=1, where the softmax is the
# constant 1) has no scale to be relative to: below this absolute floor a difference passes.
ABS_FLOOR = {1e-4: 1e-6, 2e-2: 1e-4}


def assert_close(got, want, tol, label):
    got64 = np.asarray(got, dtype=np.float64)
    want64 = np.asarray(want, dtype=np.float64)
    assert got64.shape == want64.shape, (label, got64.shape, want64.shape)
    assert np.isfinite(got64).all(), f"{label}: non-finite values in result"
    err = float(np.abs(got64 - want64).max())
    bound = tol * float(np.abs(want64).max()) + ABS_FLOOR.get(tol, 0.0)
    assert err <= bound, f"{label}: max-abs error {err:.3e} > {bound:.3e} (tol {tol:.0e} of max-abs)"
    return err / max(float(np.abs(want64).max()), 1e-30)
