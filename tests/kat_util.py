"""Helpers shared by the known-answer tests: load the reference's vectors and compare the
way the reference's own expectArraysClose does (tfjs-core/src/test_util.ts:23-39,130-138:
absolute 1e-3, NaN == NaN, +-Inf equal to themselves)."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TEST_EPSILON_FLOAT32 = 1e-3


def arr(values, shape=None):
    def conv(v):
        if isinstance(v, str):
            return {"NaN": np.nan, "Infinity": np.inf, "-Infinity": -np.inf}[v]
        return v
    a = np.array([conv(v) for v in values], dtype=np.float32)
    return a if shape is None else a.reshape(shape)


def load_kats(kind=None):
    with open(os.path.join(GOLDEN, "reference_kats.json")) as f:
        kats = json.load(f)
    return [k for k in kats if kind is None or k["kind"] == kind]


def kat_id(k):
    return k["source"].split("/")[-1] + " " + k["name"][:40]


def expect_arrays_close(actual, expected, eps=TEST_EPSILON_FLOAT32):
    actual = np.asarray(actual, dtype=np.float64).ravel()
    expected = np.asarray(expected, dtype=np.float64).ravel()
    assert actual.shape == expected.shape, (actual.shape, expected.shape)
    for i, (a, e) in enumerate(zip(actual, expected)):
        if np.isnan(a) and np.isnan(e):
            continue
        if np.isinf(e) or np.isinf(a):
            assert a == e, f"index {i}: {a} != {e}"
            continue
        assert not np.isnan(a) and not np.isnan(e) and abs(a - e) <= eps, \
            f"index {i}: actual {a} expected {e}"
