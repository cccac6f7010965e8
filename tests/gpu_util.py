"""Shared helpers of the GPU parity tests."""
import numpy as np
import pytest


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


# Tolerances stated by the task: relative Frobenius error vs the float64 oracle.
TOL_TF32 = 1e-3
TOL_3XTF32 = 1e-5
TOL_FP32 = 1e-5


@pytest.fixture(scope="module")
def ctx():
    from flutter_ml_b200 import _lib
    c = _lib.Context()
    yield c
    assert c.device_status() == 0
    c.close()
