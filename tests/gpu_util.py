"""Helpers shared by the GPU parity tests."""
import numpy as np

TOL = 1e-3  # |a - b| <= TOL * max(|b|, 1), the reference's own rule (src/kquant_dot.rs:846-851)


def assert_close(got, want, tol=TOL, what=""):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    err = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    worst = float(err.max()) if err.size else 0.0
    assert worst <= tol, f"{what}: max relative error {worst:.3e} > {tol:g} at {np.unravel_index(err.argmax(), err.shape)}"
    return worst


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
