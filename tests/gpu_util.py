"""Shared fixtures for the GPU parity tests: one cuda backend per test session."""
import numpy as np
import pytest


@pytest.fixture(scope="session")
def tf():
    import tfjs_core_b200 as tf
    assert tf.set_backend("cuda"), "cuda backend failed to initialise on a GPU machine"
    yield tf


def rel_err(got, want):
    """max |got - want| / max |want|: error relative to the tensor's largest magnitude.  An
    element-wise relative error is ill-posed for contractions: outputs near zero come from
    cancellation of K products, and even a float32 accumulation in another order misses them by
    ~1e-6 of the tensor's scale."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def ulp_diff(got, want):
    """Largest distance in float32 units in the last place."""
    a = np.asarray(got, np.float32).reshape(-1).view(np.int32).astype(np.int64)
    b = np.asarray(want, np.float32).reshape(-1).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7fffffff), a)
    b = np.where(b < 0, -(b & 0x7fffffff), b)
    return int(np.abs(a - b).max()) if a.size else 0
