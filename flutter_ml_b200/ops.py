"""Layer-level operations on device arrays, composed from the C-ABI kernels.

Each function names the reference code it stands in for.  Shapes follow the reference's
DenseLayerMatrix convention: activations are [rows x features], weights [in x out]
(lib/layertypes/denseLayer.dart:96-104).
"""
from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import ACT_BY_NAME


def dense_forward(ctx, X, W, b, act, M, N, K, Y, Z=None, precision=-1):
    """Y = act(X.W + b), optionally saving the pre-activation Z: matMul + addMatrixAndVector +
    activation (denseLayer.dart:116-125) as ONE kernel (bias and activation in the epilogue)."""
    ctx.gemm(X, W, Y, M, N, K, bias=b, preact=Z, act=act, precision=precision)


def dense_backward(ctx, X, W, saved, dY, act, M, N, K, dZ, dX=None, dW=None, db=None, accumulate=False,
                   precision=-1):
    """Gradients of dense_forward.  saved = Z for relu/gelu, Y for sigmoid/tanh.
    dZ = dY * act'(saved) and db = column sums (tensor.dart:1030, 698-704), then
    dX (+)= dZ.W^T (tensor.dart:918-924) and dW (+)= X^T.dZ (:935-941); the transposes are operand
    layout flags, nothing is copied.  db must be zeroed by the caller unless it accumulates."""
    code = ACT_BY_NAME[act]
    if code == _lib.ACT_NONE and db is None:
        dZ = dY
    else:
        ctx.call("fml_act_bwd", code, saved, dY, dZ, M, N, 0, db, launches=2 if db is not None else 1)
    beta = 1.0 if accumulate else 0.0
    if dX is not None:
        ctx.gemm(dZ, W, dX, M, K, N, transB=True, beta=beta, precision=precision)
    if dW is not None:
        ctx.gemm(X, dZ, dW, K, N, M, transA=True, beta=beta, precision=precision)
    return dZ


class DenseFwdBwdHost:
    """The dense forward+backward step driven from HOST buffers, the way the reference's FFI
    binding is used (lib/cuda/cudacaller.dart:25-60: host lists in, host list out), but with
    device buffers and pinned staging kept between calls."""

    def __init__(self, ctx, M, N, K, act="gelu", precision=-1):
        self.ctx, self.M, self.N, self.K, self.act, self.precision = ctx, M, N, K, act, precision
        e = ctx.empty
        self.A, self.B, self.bias, self.dC = e(M, K), e(K, N), e(N), e(M, N)
        self.C, self.Z, self.dZ, self.dA, self.dB, self.dbias = e(M, N), e(M, N), e(M, N), e(M, K), e(K, N), e(N)
        p = ctx.pinned
        self.h_in = {"A": p((M, K)), "B": p((K, N)), "bias": p((N,)), "dC": p((M, N))}
        self.h_out = {"C": p((M, N)), "dA": p((M, K)), "dB": p((K, N)), "dbias": p((N,))}
        self.h2d_bytes = sum(a.nbytes for a in self.h_in.values())
        self.d2h_bytes = sum(a.nbytes for a in self.h_out.values())

    def compute(self):
        c = self.ctx
        dense_forward(c, self.A, self.B, self.bias, self.act, self.M, self.N, self.K, self.C, self.Z, self.precision)
        c.zero(self.dbias)
        dense_backward(c, self.A, self.B, self.Z, self.dC, self.act, self.M, self.N, self.K, self.dZ, self.dA, self.dB,
                       self.dbias, precision=self.precision)

    def __call__(self):
        """One end-to-end step: pinned host -> device, compute, device -> pinned host."""
        c = self.ctx
        for k, dst in (("A", self.A), ("B", self.B), ("bias", self.bias), ("dC", self.dC)):
            c.upload_async(self.h_in[k], dst)
        self.compute()
        for k, src in (("C", self.C), ("dA", self.dA), ("dB", self.dB), ("dbias", self.dbias)):
            c.download_into(src, self.h_out[k])  # the last one synchronises
        return self.h_out
