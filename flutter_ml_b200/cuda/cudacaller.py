"""CudaCaller with the reference's signature (lib/cuda/cudacaller.dart:13-60), bound to the
legacy `multiplyMatrices` symbol of libflutter_ml_b200.so."""
from __future__ import annotations

from typing import List

import numpy as np

from .. import _lib


class CudaCaller:
    @staticmethod
    def matmult(A: List[float], B: List[float], m: int, k: int, n: int) -> List[float]:
        """Row-major A (m x k) times B (k x n); returns the flat m x n product as a list of
        doubles, like the Dart method (cudacaller.dart:25-26, 49-53)."""
        assert len(A) == m * k, "Matrix A has incorrect dimensions."      # cudacaller.dart:28
        assert len(B) == k * n, "Matrix B has incorrect dimensions."      # cudacaller.dart:29
        a = np.ascontiguousarray(A, dtype=np.float32)
        b = np.ascontiguousarray(B, dtype=np.float32)
        c = np.zeros(m * n, dtype=np.float32)
        lib = _lib.load()
        lib.multiplyMatrices(a.ctypes.data, b.ctypes.data, c.ctypes.data, m, k, n)
        err = lib.fml_last_error(None).decode()
        if err:
            raise _lib.FmlError(err)
        return c.astype(np.float64).tolist()
