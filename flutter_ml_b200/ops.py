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
                   precision=-1, after_dW=None):
    """Gradients of dense_forward.  saved = Z for relu/gelu, Y for sigmoid/tanh.
    dZ = dY * act'(saved) and db = column sums (tensor.dart:1030, 698-704), then
    dX (+)= dZ.W^T (tensor.dart:918-924) and dW (+)= X^T.dZ (:935-941); the transposes are operand
    layout flags, nothing is copied.  db must be zeroed by the caller unless it accumulates.  The weight gradient is
    queued first; `after_dW()` (if given) runs on the host right behind it, which is where a data-parallel caller starts
    the exchange of dW and db so that it overlaps the dX product."""
    code = ACT_BY_NAME[act]
    if code == _lib.ACT_NONE and db is None:
        dZ = dY
    else:
        ctx.call("fml_act_bwd", code, saved, dY, dZ, M, N, 0, db)
    beta = 1.0 if accumulate else 0.0
    if dW is not None:
        ctx.gemm(X, dZ, dW, K, N, M, transA=True, beta=beta, precision=precision)
    if after_dW is not None:
        after_dW()
    if dX is not None:
        ctx.gemm(dZ, W, dX, M, K, N, transB=True, beta=beta, precision=precision)
    return dZ


class GradientExchange:
    """Data-parallel exchange of a layer's weight and bias gradient, overlapped with the product that follows: the
    all-reduce (sum over ranks, NCCL) is enqueued on side stream `lane` behind everything queued so far, the persistent
    products that run beside it leave `reserve_sms` SMs free for it, and `join` makes the main stream wait for it."""

    def __init__(self, ctx, world: int, lane: int = 2, reserve_sms: int = 0, ev_start: int = 60, ev_done: int = 61,
                 overlap_rows: int = 0):
        self.ctx, self.world, self.lane, self.reserve = ctx, world, lane, reserve_sms
        self.ev_start, self.ev_done = ev_start, ev_done
        # rows of the product that follows which are computed on the reduced SM set while the exchange runs; the rest of
        # it is launched with all SMs again (0: the whole product runs on the reduced set)
        self.overlap_rows = overlap_rows

    def start(self, buf, n):
        if self.world == 1:
            return
        c, L = self.ctx, self.ctx.lib
        c.check(L.fml_event_record_on(c.h, self.ev_start, -1))
        c.check(L.fml_wait_event(c.h, self.lane, self.ev_start))
        c.check(L.fml_dp_allreduce_sum_on(c.h, self.lane, buf.ptr, n))
        c.check(L.fml_event_record_on(c.h, self.ev_done, self.lane))
        if self.reserve:
            c.check(L.fml_set_sm_reserve(c.h, self.reserve))

    def release_sms(self):
        """Later launches may use every SM again (the exchange is expected to be over by the time they start)."""
        if self.world > 1 and self.reserve:
            self.ctx.check(self.ctx.lib.fml_set_sm_reserve(self.ctx.h, 0))

    def join(self):
        if self.world == 1:
            return
        c, L = self.ctx, self.ctx.lib
        self.release_sms()
        c.check(L.fml_wait_event(c.h, -1, self.ev_done))


class DenseFwdBwdHost:
    """The dense forward+backward step driven from HOST buffers, the way the reference's FFI
    binding is used (lib/cuda/cudacaller.dart:25-60: host lists in, host list out), but with
    device buffers and pinned staging kept between calls."""

    def __init__(self, ctx, M, N, K, act="gelu", precision=-1, exchange=None):
        self.ctx, self.M, self.N, self.K, self.act, self.precision = ctx, M, N, K, act, precision
        self.exchange = exchange     # GradientExchange or None: sums dB and dbias over the data-parallel ranks
        e = ctx.empty
        self.A, self.B, self.bias, self.dC = e(M, K), e(K, N), e(N), e(M, N)
        self.C, self.Z, self.dZ, self.dA = e(M, N), e(M, N), e(M, N), e(M, K)
        self._gb_off = (K * N + 3) & ~3          # bias gradient at a 16-byte aligned offset behind the weight gradient
        self.grads = e(self._gb_off + N)         # side by side: one exchange
        self.dB, self.dbias = self.grads.view(0, (K, N)), self.grads.view(self._gb_off, (N,))
        p = ctx.pinned
        self.h_in = {"A": p((M, K)), "B": p((K, N)), "bias": p((N,)), "dC": p((M, N))}
        self.h_out = {"C": p((M, N)), "dA": p((M, K)), "dB": p((K, N)), "dbias": p((N,))}
        self.h2d_bytes = sum(a.nbytes for a in self.h_in.values())
        self.d2h_bytes = sum(a.nbytes for a in self.h_out.values())

    def compute(self, d=None):
        """Forward, dZ + dbias, dW, [exchange of dW and dbias started], dA, [exchange joined] on buffer set `d`."""
        c = self.ctx
        d = d or {k: getattr(self, k) for k in ("A", "B", "bias", "dC", "C", "Z", "dZ", "dA", "dB", "dbias", "grads")}
        dense_forward(c, d["A"], d["B"], d["bias"], self.act, self.M, self.N, self.K, d["C"], d["Z"], self.precision)
        c.zero(d["dbias"])
        ex = self.exchange
        M, N, K = self.M, self.N, self.K
        split = ex.overlap_rows if (ex and ex.world > 1 and 0 < ex.overlap_rows < M) else 0
        dense_backward(c, d["A"], d["B"], d["Z"], d["dC"], self.act, M, N, K, d["dZ"], None if split else d["dA"], d["dB"],
                       d["dbias"], precision=self.precision,
                       after_dW=(lambda: ex.start(d["grads"], d["grads"].size)) if ex else None)
        if split:
            # dA in two row blocks: the first beside the exchange on the reduced SM set, the second on all SMs
            c.gemm(d["dZ"], d["B"], d["dA"], split, K, N, transB=True, precision=self.precision)
            ex.release_sms()
            c.gemm(d["dZ"].view(split * N, (M - split, N)), d["B"], d["dA"].view(split * K, (M - split, K)), M - split, K, N,
                   transB=True, precision=self.precision)
        if ex:
            ex.join()

    def pipelined(self, steps: int):
        """`steps` end-to-end steps with the copies on two side streams and two sets of device buffers,
        so the upload of step s+1, the kernels of step s and the download of step s-1 overlap (PCIe is
        full duplex).  Same bytes per step as __call__; every step still uploads and downloads everything."""
        c, L = self.ctx, self.ctx.lib
        if not hasattr(self, "_sets"):
            e, (M, N, K) = c.empty, (self.M, self.N, self.K)
            second = dict(A=e(M, K), B=e(K, N), bias=e(N), dC=e(M, N), C=e(M, N), Z=e(M, N), dZ=e(M, N), dA=e(M, K),
                          grads=e(self._gb_off + N))
            second["dB"], second["dbias"] = second["grads"].view(0, (K, N)), second["grads"].view(self._gb_off, (N,))
            first = {k: getattr(self, k) for k in second}
            self._sets = [first, second]
        EV_UP, EV_COMP, EV_DOWN = 40, 42, 44     # event slots, +0/+1 per buffer set
        chk = c.check

        def upload(s):
            b = s % 2
            if s >= 2:
                chk(L.fml_wait_event(c.h, 0, EV_COMP + b))   # the kernels of step s-2 have read this set
            for k in ("A", "B", "bias", "dC"):
                chk(L.fml_lane_h2d(c.h, 0, self._sets[b][k].ptr, self.h_in[k].ctypes.data, self.h_in[k].size))
            chk(L.fml_event_record_on(c.h, EV_UP + b, 0))

        upload(0)
        for s in range(steps):
            b = s % 2
            d = self._sets[b]
            if s + 1 < steps:
                upload(s + 1)
            chk(L.fml_wait_event(c.h, -1, EV_UP + b))
            if s >= 2:
                chk(L.fml_wait_event(c.h, -1, EV_DOWN + b))  # the download of step s-2 has drained this set
            self.compute(d)
            chk(L.fml_event_record_on(c.h, EV_COMP + b, -1))
            chk(L.fml_wait_event(c.h, 1, EV_COMP + b))
            for k in ("C", "dA", "dB", "dbias"):
                chk(L.fml_lane_d2h(c.h, 1, self.h_out[k].ctypes.data, d[k].ptr, d[k].size))
            chk(L.fml_event_record_on(c.h, EV_DOWN + b, 1))
        chk(L.fml_lane_sync(c.h, 1))
        chk(L.fml_lane_sync(c.h, 0))
        c.sync()
        return self.h_out

    def __call__(self):
        """One end-to-end step: pinned host -> device, compute, device -> pinned host."""
        c = self.ctx
        for k, dst in (("A", self.A), ("B", self.B), ("bias", self.bias), ("dC", self.dC)):
            c.upload_async(self.h_in[k], dst)
        self.compute()
        for k, src in (("C", self.C), ("dA", self.dA), ("dB", self.dB), ("dbias", self.dbias)):
            c.download_into(src, self.h_out[k])  # the last one synchronises
        return self.h_out
