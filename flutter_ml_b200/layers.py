"""Layers with the reference's names and call protocol (lib/layertypes, lib/transformer).

`Layer.call` builds on first use and then runs `forward` (lib/layertypes/layer.dart:80-85).
Every layer accepts a batch of sequences flattened into rows ([n_seq * seq_len, features]); a
single sequence (n_seq = 1) is exactly the reference's `Tensor<Matrix>` input.  The reference
draws its initial weights from an unseeded `Random()`; here each layer takes an explicit
`seed` and uses the counter-based generator of `synth`.
"""
from __future__ import annotations

import math
from typing import List, Optional

import numpy as np

from . import synth
from . import tensor as T
from .tensor import Tensor


class Layer:
    """lib/layertypes/layer.dart:48-86."""

    name = "Layer"

    def __init__(self):
        self._built = False

    @property
    def parameters(self) -> List[Tensor]:
        return []

    def build(self, x):
        self._built = True

    def forward(self, x):
        raise NotImplementedError

    def call(self, x):
        if not self._built:
            self.build(x)
        return self.forward(x)

    __call__ = call


class DenseLayerMatrix(Layer):
    """act(X.W + b), W [in x out] (lib/layertypes/denseLayer.dart:76-126); He-normal weights
    (:93-100), zero bias."""

    name = "dense_matrix"

    def __init__(self, outputSize: int, activation: Optional[str] = None, seed: int = 0, weights=None, bias=None,
                 precision: int = -1):
        super().__init__()
        self.outputSize, self.activation, self.seed, self.precision = outputSize, activation, seed, precision
        self._w0, self._b0 = weights, bias
        self.weights: Optional[Tensor] = None
        self.biases: Optional[Tensor] = None

    @property
    def parameters(self):
        return [self.weights, self.biases]

    def build(self, x: Tensor):
        fan_in = x.shape[1]
        w = self._w0 if self._w0 is not None else synth.normal(self.seed, 0, (fan_in, self.outputSize), math.sqrt(2.0 / fan_in))
        b = self._b0 if self._b0 is not None else np.zeros(self.outputSize, dtype=np.float32)
        self.weights, self.biases = Tensor(w, x.ctx), Tensor(b, x.ctx)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        if self.activation in T.ACT2_BY_NAME:
            # LeakyReLU / ELU / Swish / Mish are not epilogue functors of the contraction: bias-fused product, then
            # the streaming activation (lib/layertypes/denseLayer.dart:116-125 applies them the same way)
            z = T.denseMatrix(x, self.weights, self.biases, None, self.precision)
            return T.ACT2_BY_NAME[self.activation](z)
        return T.denseMatrix(x, self.weights, self.biases, self.activation, self.precision)


class DenseLayer(DenseLayerMatrix):
    """The vector form act(W.x + b) with W stored [out x in] (lib/layertypes/denseLayer.dart:15-64: He-normal
    weights :18-25, matVecMul + addVector :42).  The input vector is taken as a [1 x in] row (a flat [in] tensor is
    reshaped), the product runs as x.W^T through the same fused dense node as the matrix form — the transpose is
    a node of its own, so the gradient arrives in the [out x in] layout the reference's optimizer sees — and
    the output is the [1 x out] row."""

    name = "dense"

    def build(self, x: Tensor):
        fan_in = x.shape[-1]
        w = self._w0 if self._w0 is not None else synth.normal(self.seed, 0, (self.outputSize, fan_in), math.sqrt(2.0 / fan_in))
        b = self._b0 if self._b0 is not None else np.zeros(self.outputSize, dtype=np.float32)
        self.weights, self.biases = Tensor(w, x.ctx), Tensor(b, x.ctx)
        Layer.build(self, x)

    def forward(self, x: Tensor) -> Tensor:
        if len(x.shape) == 1:
            row = Tensor(x.value.reshape(1, x.shape[0]), x.ctx)
            if x.creator is not None or x.grad is not None:
                raise ValueError("DenseLayer: pass the input vector as a [1 x in] row when it needs a gradient")
            x = row
        wt = T.transpose(self.weights)
        if self.activation in T.ACT2_BY_NAME:
            return T.ACT2_BY_NAME[self.activation](T.denseMatrix(x, wt, self.biases, None, self.precision))
        return T.denseMatrix(x, wt, self.biases, self.activation, self.precision)


class Conv2DLayer(Layer):
    """lib/layertypes/conv2d.dart:11-75: `outChannels` square kernels over a single-channel input, one scalar bias
    each, padding 'valid' or 'same'.  The reference keeps a list of kernel matrices; here they are the rows of one
    [outChannels x kernelSize^2] tensor so that the layer is one launch.  Input [n_img, H, W] -> output [n_img, outChannels, OH, OW]; a single matrix [H, W]
    -> [outChannels, OH, OW] like the reference's Tensor3D.  Initial kernels uniform(+-sqrt(2 / k^2)) as conv2d.dart:37-45, biases 0."""

    name = "conv2d_layer"

    def __init__(self, outChannels: int, kernelSize: int, padding: str = "valid", seed: int = 0, kernels=None, biases=None):
        super().__init__()
        self.outChannels, self.kernelSize, self.padding, self.seed = outChannels, kernelSize, padding, seed
        self._k0, self._b0 = kernels, biases
        self.kernels: Optional[Tensor] = None
        self.biases: Optional[Tensor] = None

    @property
    def parameters(self):
        return [self.kernels, self.biases]

    def build(self, x: Tensor):
        k2 = self.kernelSize * self.kernelSize
        a = math.sqrt(2.0 / k2)
        k = self._k0 if self._k0 is not None else synth.uniform(self.seed, 0, (self.outChannels, k2), -a, a)
        b = self._b0 if self._b0 is not None else np.zeros(self.outChannels, dtype=np.float32)
        self.kernels = Tensor(np.asarray(k, dtype=np.float32).reshape(self.outChannels, k2), x.ctx)
        self.biases = Tensor(b, x.ctx)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        return T.conv2dBatch(x, self.kernels, self.biases, self.kernelSize, self.kernelSize, self.padding)


class LSTMLayer(Layer):
    """LSTMLayer (lib/layertypes/lstmLayer.dart:37-151): gates f, i, c~, o over the concatenated [h_{t-1}, x_t]
    (:119), output = the last hidden state (:149).

    Input: one sequence [T x I] (the reference's Tensor<Matrix>) or a time-major batch [T x B x I]; output
    [B x H] (B = 1 for one sequence).  The four gate matrices [H x (H+I)] live in one [4H x (H+I)] buffer, the
    four biases in one [4H] buffer, so that the whole recurrence runs in the library's fused LSTM kernels;
    `parameters` hands out the eight tensors of the reference in its order (W_f, b_f, W_i, b_i, W_c, b_c, W_o,
    b_o, :41) as views into those buffers.  Initial weights U(+-1/sqrt(H+I)) (:80) from the seeded generator
    unless `weights` ([4H x (H+I)]) / `bias` ([4H]) are given."""
    name = "lstm"

    def __init__(self, hiddenSize: int, seed: int = 0, weights=None, bias=None):
        super().__init__()
        self.hiddenSize, self.seed, self._w0, self._b0 = hiddenSize, seed, weights, bias

    @property
    def parameters(self):
        return self._params

    def build(self, x: Tensor):
        H, I = self.hiddenSize, x.shape[-1]
        ctx = x.ctx
        a = 1.0 / math.sqrt(H + I)
        w = self._w0 if self._w0 is not None else synth.uniform(self.seed, 0, (4 * H, H + I), -a, a)
        b = self._b0 if self._b0 is not None else np.zeros(4 * H, dtype=np.float32)
        self.W, self.b = ctx.upload(np.asarray(w, np.float32)), ctx.upload(np.asarray(b, np.float32))
        self.dW, self.db = ctx.zeros(4 * H, H + I), ctx.zeros(4 * H)
        self._params = []
        for g in range(4):
            for buf, grad, off, shape in ((self.W, self.dW, g * H * (H + I), (H, H + I)), (self.b, self.db, g * H, (H,))):
                t = Tensor(buf.view(off, shape), ctx)
                t.grad = grad.view(off, shape)
                self._params.append(t)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        import ctypes
        from . import _lib
        ctx, H = x.ctx, self.hiddenSize
        Tn, B, I = (x.shape[0], 1, x.shape[1]) if len(x.shape) == 2 else x.shape
        d = _lib.LstmDesc()
        d.T, d.B, d.I, d.H = Tn, B, I, H
        saved = dict(gates=ctx.empty(Tn, B, 4 * H), cells=ctx.empty(Tn + 1, B, H), hs=ctx.empty(Tn + 1, B, H),
                     xproj=ctx.empty(Tn * B, 4 * H))
        d.W, d.b, d.x = self.W.ptr, self.b.ptr, x.value.ptr
        for k, v in saved.items():
            setattr(d, k, v.ptr)
        ctx.check(ctx.lib.fml_lstm_fwd(ctx.h, ctypes.byref(d)))
        ctx.launches += 3
        out = Tensor(saved["hs"].view(Tn * B * H, (B, H)), ctx)

        def bw(_keep=saved):   # the descriptor points into the saved buffers: they live as long as this closure
            scratch = ctx.empty(Tn * B * 4 * H + 2 * B * H)
            dx = None
            if x.creator is not None or x.grad is not None:    # someone upstream wants the input gradient
                dx = ctx.empty(*x.shape)
            ctx.check(ctx.lib.fml_lstm_bwd(ctx.h, ctypes.byref(d), out.grad.ptr, self.dW.ptr, self.db.ptr,
                                           dx.ptr if dx is not None else None, scratch.ptr))
            ctx.launches += 2 * Tn + 9
            if dx is not None:
                x._add_grad(dx, alias=True)
        out.creator = T.Node([x] + self._params, bw, "lstm", cost=8 * Tn * B * H * (H + I))
        return out


class MultiTierLSTMLayer(Layer):
    """MultiTierLSTMLayer (lib/layertypes/multilstm.dart:14-208): a stack of LSTM tiers on different clocks.

    Tier 0 runs at every step on [h_0, c_1, ..., c_{n-1}, x_t] (its own hidden state, the CELL states of all higher tiers
    as context, the input: :137-150); tier i >= 1 runs when (step + 1) is a multiple of the product of the first i clock
    cycles (:155), on [h_i, h_{i-1}] with h_{i-1} as just updated in the same step (:157).  Output: the last hidden state
    of tier 0 (:166).  All states start at zero (:117-121).

    Input: one sequence [T x I] or a time-major batch [T x B x I]; output [B x H].  Per tier the four gate matrices
    [H x combined] of the reference live in one [4H x combined] buffer (gate blocks f, i, c~, o), the biases in one [4H]
    buffer; `parameters` hands out the reference's tensors in its order, tier by tier (W_f, b_f, W_i, b_i, W_c, b_c, W_o,
    b_o, :44-52), as views.  A cell update is: one product per input block into the [B x 4H] pre-activations (the first
    with the bias in its epilogue, the others accumulating; the concatenated input of the reference never exists; the
    input's block of tier 0 is one product over all time steps), then fml_lstm_cell_fwd.  Backward runs the recorded updates in reverse with fml_lstm_cell_bwd and the transposed
    products; gradients of states that feed several later updates accumulate in place.  Initial weights
    U(+-sqrt(1/fanIn)) (:66-77) from the seeded generator unless `weights` / `biases` (one array per tier) are given."""
    name = "multitier_lstm"

    def __init__(self, hiddenSize: int, tierClockCycles, seed: int = 0, weights=None, biases=None):
        super().__init__()
        self.hiddenSize, self.tierClockCycles = hiddenSize, list(tierClockCycles)
        self.numTiers = len(self.tierClockCycles) + 1
        self.cumulativeClockCycles, prod = [], 1
        for c in self.tierClockCycles:
            if c < 1:
                raise ValueError("clock cycles must be positive")
            prod *= c
            self.cumulativeClockCycles.append(prod)
        self.seed, self._w0, self._b0 = seed, weights, biases

    def _fires(self, tier: int, step: int) -> bool:
        return (step + 1) % self.cumulativeClockCycles[tier - 1] == 0      # multilstm.dart:155

    def _combined(self, tier: int, I: int) -> int:
        H = self.hiddenSize
        return H + (self.numTiers - 1) * H + I if tier == 0 else 2 * H     # multilstm.dart:82-88

    @property
    def parameters(self):
        return self._params

    def build(self, x: Tensor):
        H, I, ctx = self.hiddenSize, x.shape[-1], x.ctx
        self.W, self.b, self.dW, self.db, self._params = [], [], [], [], []
        for i in range(self.numTiers):
            comb = self._combined(i, I)
            a = math.sqrt(1.0 / comb)
            w = self._w0[i] if self._w0 is not None else synth.uniform(self.seed, 10 + i, (4 * H, comb), -a, a)
            b = self._b0[i] if self._b0 is not None else np.zeros(4 * H, dtype=np.float32)
            w = np.ascontiguousarray(w, np.float32)
            if w.shape != (4 * H, comb):
                raise ValueError(f"tier {i}: weights must be [4H x {comb}]")
            self.W.append(ctx.upload(w))
            self.b.append(ctx.upload(np.asarray(b, np.float32)))
            self.dW.append(ctx.zeros(4 * H, comb))
            self.db.append(ctx.zeros(4 * H))
            for g in range(4):
                for buf, grad, off, shape in ((self.W[i], self.dW[i], g * H * comb, (H, comb)), (self.b[i], self.db[i], g * H, (H,))):
                    t = Tensor(buf.view(off, shape), ctx)
                    t.grad = grad.view(off, shape)
                    self._params.append(t)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        ctx, H, n = x.ctx, self.hiddenSize, self.numTiers
        Tn, B, I = (x.shape[0], 1, x.shape[1]) if len(x.shape) == 2 else x.shape
        zero = ctx.zeros(B, H)                       # every initial state (read only)
        h, c = [zero] * n, [zero] * n
        records = []                                 # (tier, step, [(input block, width, first column)], c_prev, gates, c_new, h_new)
        comb0 = self._combined(0, I)
        # The input's share of tier 0's pre-activations does not depend on the recurrence: one product for all steps
        # (bias in its epilogue); the recurrent blocks are added step by step.
        pre_all = ctx.empty(Tn * B, 4 * H)
        ctx.gemm(x.value, self.W[0].view(n * H, (4 * H, I)), pre_all, Tn * B, 4 * H, I, transB=True, ldb=comb0, bias=self.b[0])

        def update(tier, step, blocks, pre=None):
            comb = self._combined(tier, I)
            first = pre is None
            if first:
                pre = ctx.empty(B, 4 * H)
            for k, (arr, w, col) in enumerate(blocks):
                if arr is zero and not (first and k == 0):
                    continue                          # an initial state adds nothing
                ctx.gemm(arr, self.W[tier].view(col, (4 * H, w)), pre, B, 4 * H, w, transB=True, ldb=comb,
                         bias=self.b[tier] if (first and k == 0) else None, beta=0.0 if (first and k == 0) else 1.0)
            gates, c_new, h_new = ctx.empty(B, 4 * H), ctx.empty(B, H), ctx.empty(B, H)
            ctx.call("fml_lstm_cell_fwd", pre, c[tier], gates, c_new, h_new, B, H)
            records.append((tier, step, blocks, c[tier], gates, c_new, h_new))
            h[tier], c[tier] = h_new, c_new

        for t in range(Tn):
            blocks = [(h[0], H, 0)] + [(c[j], H, j * H) for j in range(1, n)]
            update(0, t, blocks, pre_all.view(t * B * 4 * H, (B, 4 * H)))
            for i in range(1, n):
                if self._fires(i, t):
                    update(i, t, [(h[i], H, 0), (h[i - 1], H, H)])
        out = Tensor(h[0], ctx)
        want_dx = x.creator is not None or x.grad is not None

        def bw():
            grads = {id(out.value): out.grad}

            def grad_of(arr):
                g = grads.get(id(arr))
                if g is None:
                    g = grads[id(arr)] = ctx.zeros(B, H)
                return g
            dpre_all = ctx.zeros(Tn * B, 4 * H)       # tier 0's pre-activation gradients of all steps (zero where none flows)
            for tier, step, blocks, c_prev, gates, c_new, h_new in reversed(records):
                dh, dc = grads.get(id(h_new)), grads.get(id(c_new))
                if dh is None and dc is None:
                    continue                          # nothing downstream read this update
                comb = self._combined(tier, I)
                dpre = dpre_all.view(step * B * 4 * H, (B, 4 * H)) if tier == 0 else ctx.empty(B, 4 * H)
                if c_prev is zero:
                    dcp, acc = ctx.empty(B, H), 0     # gradient of the initial state: formed, not used
                else:
                    acc = 1 if id(c_prev) in grads else 0
                    dcp = grads[id(c_prev)] if acc else grads.setdefault(id(c_prev), ctx.empty(B, H))
                ctx.call("fml_lstm_cell_bwd", gates, c_prev, c_new, dh, dc, dpre, dcp, acc, B, H)
                if tier > 0:
                    ctx.call("fml_col_sum", dpre, self.db[tier], B, 4 * H, 1)
                for arr, w, col in blocks:
                    if arr is zero:
                        continue                      # no weight gradient from a zero input, no gradient into it
                    ctx.gemm(dpre, arr, self.dW[tier].view(col, (4 * H, w)), 4 * H, w, B, transA=True, ldc=comb, beta=1.0)
                    ctx.gemm(dpre, self.W[tier].view(col, (4 * H, w)), grad_of(arr), B, w, 4 * H, ldb=comb, beta=1.0)
            # the input's share, all steps at once
            ctx.call("fml_col_sum", dpre_all, self.db[0], Tn * B, 4 * H, 1)
            ctx.gemm(dpre_all, x.value, self.dW[0].view(n * H, (4 * H, I)), 4 * H, I, Tn * B, transA=True, ldc=comb0, beta=1.0)
            if want_dx:
                dx = ctx.empty(*x.shape)
                ctx.gemm(dpre_all, self.W[0].view(n * H, (4 * H, I)), dx, Tn * B, I, 4 * H, ldb=comb0)
                x._add_grad(dx, alias=True)
        out.creator = T.Node([x] + self._params, bw, self.name, cost=8 * len(records) * B * H * 2 * H)
        return out


class DualLSTMLayer(MultiTierLSTMLayer):
    """DualLSTMLayer (lib/layertypes/duallstm.dart:26-175): two tiers; the higher one runs when step > 0 and (step + 1) is
    a multiple of `lowerTierClockCycle` (:145), on [h_higher, h_lower] (:149); the lower one at every step on
    [h_lower, c_higher, x_t] (:116-117).  Parameters in the reference's order: the lower tier's eight, then the higher
    tier's (:43-46)."""
    name = "duallstm"

    def __init__(self, hiddenSize: int, lowerTierClockCycle: int = 7, seed: int = 0, weights=None, biases=None):
        super().__init__(hiddenSize, [lowerTierClockCycle], seed=seed, weights=weights, biases=biases)
        self.lowerTierClockCycle = lowerTierClockCycle

    def _fires(self, tier: int, step: int) -> bool:
        return step > 0 and (step + 1) % self.lowerTierClockCycle == 0


class ConvLSTMLayer(Layer):
    """ConvLSTMLayer (lib/layertypes/convlstmLayer.dart:37-159): an LSTM whose gates are single-channel convolutions with
    'same' padding over the frame and over the hidden map, one bias MATRIX per gate (:83-96); hidden and cell states are
    [H x W] maps, the output is the last hidden map (:157).  `hiddenFilters` is accepted and, as in the reference, unused.

    Input: one sequence of frames [T x H x W] or a time-major batch [T x B x H x W]; output [H x W] or [B x H x W].  The four
    input kernels are the rows of one [4 x k^2] tensor, likewise the four hidden kernels, the four bias matrices one
    [4 x H*W] buffer; `parameters` hands out the reference's twelve tensors in its order (K_xf, K_hf, b_f, K_xi, ... :51-56)
    as views.  A step is two launches of the batched convolution (all four gates of a frame at once: their output
    [B x 4 x H*W] IS the gate-blocked pre-activation layout), the bias, and fml_lstm_cell_fwd with one "hidden unit" per
    pixel; backward fml_lstm_cell_bwd and the convolution's backward, which adds into the kernel gradients.  Initial kernels
    U(+-sqrt(1/k^2)) (:66-76) from the seeded generator unless given."""
    name = "conv_lstm"

    def __init__(self, hiddenFilters: int, kernelSize: int, seed: int = 0, kernels_x=None, kernels_h=None, biases=None):
        super().__init__()
        if kernelSize % 2 == 0:
            raise ValueError("'same' padding needs an odd kernel size")
        self.hiddenFilters, self.kernelSize, self.seed = hiddenFilters, kernelSize, seed
        self._kx0, self._kh0, self._b0 = kernels_x, kernels_h, biases

    @property
    def parameters(self):
        return self._params

    def build(self, x: Tensor):
        k2, ctx = self.kernelSize ** 2, x.ctx
        Hh, Ww = x.shape[-2], x.shape[-1]
        a = math.sqrt(1.0 / k2)
        kx = self._kx0 if self._kx0 is not None else synth.uniform(self.seed, 20, (4, k2), -a, a)
        kh = self._kh0 if self._kh0 is not None else synth.uniform(self.seed, 21, (4, k2), -a, a)
        b = self._b0 if self._b0 is not None else np.zeros((4, Hh * Ww), dtype=np.float32)
        self.Kx = ctx.upload(np.asarray(kx, np.float32).reshape(4, k2))
        self.Kh = ctx.upload(np.asarray(kh, np.float32).reshape(4, k2))
        self.b = ctx.upload(np.asarray(b, np.float32).reshape(4 * Hh * Ww))
        self.dKx, self.dKh, self.db = ctx.zeros(4, k2), ctx.zeros(4, k2), ctx.zeros(4 * Hh * Ww)
        self._params = []
        k = self.kernelSize
        for g in range(4):
            for buf, grad, off, shape in ((self.Kx, self.dKx, g * k2, (k, k)), (self.Kh, self.dKh, g * k2, (k, k)),
                                          (self.b, self.db, g * Hh * Ww, (Hh, Ww))):
                t = Tensor(buf.view(off, shape), ctx)
                t.grad = grad.view(off, shape)
                self._params.append(t)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        ctx, k = x.ctx, self.kernelSize
        single = len(x.shape) == 3
        Tn, B, Hh, Ww = (x.shape[0], 1, x.shape[1], x.shape[2]) if single else x.shape
        P, pad = Hh * Ww, (k - 1) // 2
        cargs = (B, Hh, Ww, 4, k, k, pad)
        zero = ctx.zeros(B, P)
        h, c = zero, zero
        records = []
        for t in range(Tn):
            x_t = x.value.view(t * B * P, (B, P))
            pre, hc = ctx.empty(B, 4 * P), ctx.empty(B, 4 * P)
            ctx.call("fml_conv2d_fwd", x_t, self.Kx, None, pre, *cargs)
            if h is not zero:
                ctx.call("fml_conv2d_fwd", h, self.Kh, None, hc, *cargs)
                ctx.call("fml_axpy", 1.0, hc, pre, B * 4 * P)
            ctx.call("fml_add_bias", pre, self.b, pre, B, 4 * P)
            gates, c_new, h_new = ctx.empty(B, 4 * P), ctx.empty(B, P), ctx.empty(B, P)
            ctx.call("fml_lstm_cell_fwd", pre, c, gates, c_new, h_new, B, P)
            records.append((t, h, c, gates, c_new, h_new))
            h, c = h_new, c_new
        out = Tensor(h.view(0, (Hh, Ww) if single else (B, Hh, Ww)), ctx)
        want_dx = x.creator is not None or x.grad is not None

        def bw():
            dh, dc = out.grad, None                   # gradients arriving at the states of the step being undone
            dx = ctx.zeros(*x.shape) if want_dx else None
            for t, h_prev, c_prev, gates, c_new, h_new in reversed(records):
                dpre, dc_prev = ctx.empty(B, 4 * P), ctx.empty(B, P)
                ctx.call("fml_lstm_cell_bwd", gates, c_prev, c_new, dh, dc, dpre, dc_prev, 0, B, P)
                ctx.call("fml_col_sum", dpre, self.db, B, 4 * P, 1)
                x_t = x.value.view(t * B * P, (B, P))
                ctx.call("fml_conv2d_bwd", x_t, self.Kx, dpre, dx.view(t * B * P, (B, P)) if dx is not None else None, self.dKx, None,
                         *cargs, launches=2)
                if h_prev is zero:
                    break                             # the first step: no hidden map before it
                dh_prev = ctx.zeros(B, P)
                ctx.call("fml_conv2d_bwd", h_prev, self.Kh, dpre, dh_prev, self.dKh, None, *cargs, launches=2)
                dh, dc = dh_prev, dc_prev
            if dx is not None:
                x._add_grad(dx, alias=True)
        out.creator = T.Node([x] + self._params, bw, self.name, cost=2 * Tn * B * 8 * P * k * k)
        return out


class GeneralizedChainedScaleLayer(Layer):
    """GeneralizedChainedScaleLayer (lib/layertypes/trendmodelLayer.dart:42-218): a chain of LSTMs over coarser and coarser
    summaries of the past.  Level i + 1 of the data is tanh(aggW_i . [grain_i consecutive rows of level i, flattened] +
    aggB_i) for every complete chunk (:146-158); the LSTM of the highest level runs first over (at most) its last 10
    summaries, its final hidden state initialises the hidden state of the LSTM one level down (cell state zero again),
    and so on down to level 0, which reads the last `finalSequenceLength` raw rows (:163-178).  Output: the last hidden
    state of level 0.

    Input: one sequence [T x I] or a batch-major batch [B x T x I] (consecutive rows of a sequence are contiguous, so a
    chunk is one row of a [chunks x grain*I] view and every aggregation level is one product with the tanh in its
    epilogue per sequence); output [H] / [B x H].  Every LSTM step is the input's share (one product per tier and sequence
    for all its steps, bias in the epilogue) plus h . Wh^T accumulated into it, then fml_lstm_cell_fwd on the whole batch.
    `parameters` in the reference's order (:70-84): per tier W_f, b_f, W_i, b_i, W_c, b_c, W_o, b_o (views of one
    [4H x (H+I)] / [4H] buffer, columns [h | x] as in `concatenate(h, x_t)` :193), then aggW_i, aggB_i per level."""
    name = "generalized_chained_scale"
    HIGHER_TIER_LOOKBACK = 10      # trendmodelLayer.dart:168

    def __init__(self, hiddenSize: int, grainingSizes, finalSequenceLength: int = 7, seed: int = 0, lstm_weights=None, lstm_biases=None,
                 agg_weights=None, agg_biases=None):
        super().__init__()
        self.hiddenSize, self.grainingSizes, self.finalSequenceLength = hiddenSize, list(grainingSizes), finalSequenceLength
        self.numTiers = len(self.grainingSizes) + 1
        self.seed, self._w0, self._b0, self._aw0, self._ab0 = seed, lstm_weights, lstm_biases, agg_weights, agg_biases

    @property
    def parameters(self):
        return self._params

    def build(self, x: Tensor):
        H, I, ctx = self.hiddenSize, x.shape[-1], x.ctx
        Z = H + I
        self.W, self.b, self.dW, self.db, self.aW, self.ab, self.daW, self.dab = [], [], [], [], [], [], [], []
        self._params = []
        a = math.sqrt(1.0 / Z)
        for i in range(self.numTiers):
            w = self._w0[i] if self._w0 is not None else synth.uniform(self.seed, 30 + i, (4 * H, Z), -a, a)
            b = self._b0[i] if self._b0 is not None else np.zeros(4 * H, dtype=np.float32)
            self.W.append(ctx.upload(np.ascontiguousarray(w, np.float32).reshape(4 * H, Z)))
            self.b.append(ctx.upload(np.asarray(b, np.float32)))
            self.dW.append(ctx.zeros(4 * H, Z))
            self.db.append(ctx.zeros(4 * H))
            for g in range(4):
                for buf, grad, off, shape in ((self.W[i], self.dW[i], g * H * Z, (H, Z)), (self.b[i], self.db[i], g * H, (H,))):
                    t = Tensor(buf.view(off, shape), ctx)
                    t.grad = grad.view(off, shape)
                    self._params.append(t)
        for i, grain in enumerate(self.grainingSizes):
            fan = grain * I
            aa = math.sqrt(1.0 / fan)
            w = self._aw0[i] if self._aw0 is not None else synth.uniform(self.seed, 40 + i, (I, fan), -aa, aa)
            b = self._ab0[i] if self._ab0 is not None else np.zeros(I, dtype=np.float32)
            wt, bt = Tensor(np.ascontiguousarray(w, np.float32).reshape(I, fan), ctx), Tensor(np.asarray(b, np.float32), ctx)
            wt.zeroGrad()
            bt.zeroGrad()
            self.aW.append(wt)
            self.ab.append(bt)
            self._params += [wt, bt]
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        ctx, H, n = x.ctx, self.hiddenSize, self.numTiers
        single = len(x.shape) == 2
        B, T0, I = (1,) + tuple(x.shape) if single else x.shape
        Z = H + I
        if T0 < self.finalSequenceLength:
            raise ValueError("the sequence is shorter than finalSequenceLength")
        # ---- aggregation: level i + 1 from level i, every sequence one product with the tanh in its epilogue
        data, lens = [x.value], [T0]
        for i, grain in enumerate(self.grainingSizes):
            cnt = lens[i] // grain                    # complete chunks only (trendmodelLayer.dart:150)
            S = ctx.empty(B, max(cnt, 1), I)
            for bq in range(B if cnt else 0):
                ctx.gemm(data[i].view(bq * lens[i] * I, (cnt, grain * I)), self.aW[i].value, S.view(bq * cnt * I, (cnt, I)), cnt, I, grain * I,
                         transB=True, bias=self.ab[i].value, act="tanh")
            data.append(S)
            lens.append(cnt)
        # ---- the chain of LSTMs, highest level first
        zero = ctx.zeros(B, H)
        context = zero
        tiers = []                                    # per tier, in the order run: (i, L, first row, xproj, [(h_prev, c_prev, gates, c_new, h_new)])
        for i in range(n - 1, -1, -1):
            look = self.finalSequenceLength if i == 0 else self.HIGHER_TIER_LOOKBACK
            L = min(lens[i], look)
            first = lens[i] - L
            if L == 0:
                tiers.append((i, 0, 0, None, []))
                continue
            xproj = ctx.empty(L, B, 4 * H)            # the input's share of every step's pre-activations, bias included
            for bq in range(B):
                ctx.gemm(data[i].view((bq * lens[i] + first) * I, (L, I)), self.W[i].view(H, (4 * H, I)), xproj.view(bq * 4 * H, (L, 4 * H)),
                         L, 4 * H, I, transB=True, ldb=Z, ldc=B * 4 * H, bias=self.b[i])
            h, c, steps = context, zero, []
            for l in range(L):
                pre = xproj.view(l * B * 4 * H, (B, 4 * H))
                if h is not zero:
                    ctx.gemm(h, self.W[i].view(0, (4 * H, H)), pre, B, 4 * H, H, transB=True, ldb=Z, beta=1.0)
                gates, c_new, h_new = ctx.empty(B, 4 * H), ctx.empty(B, H), ctx.empty(B, H)
                ctx.call("fml_lstm_cell_fwd", pre, c, gates, c_new, h_new, B, H)
                steps.append((h, c, gates, c_new, h_new))
                h, c = h_new, c_new
            tiers.append((i, L, first, xproj, steps))
            context = h
        out = Tensor(context.view(0, (H,)) if single else context, ctx)
        want_dx = x.creator is not None or x.grad is not None

        def bw():
            ddata = [None] * n                        # gradient of every level of the data, allocated when first needed

            def grad_level(i):
                if ddata[i] is None:
                    ddata[i] = ctx.zeros(B, max(lens[i], 1), I)
                return ddata[i]
            dctx = out.grad                           # gradient of the context handed down the chain
            for i, L, first, xproj, steps in reversed(tiers):      # level 0 ran last
                if L == 0 or dctx is None:
                    continue
                dpre_all = ctx.empty(L, B, 4 * H)
                dh, dc = dctx, None
                for l in range(L - 1, -1, -1):
                    h_prev, c_prev, gates, c_new, h_new = steps[l]
                    dpre, dc_prev = dpre_all.view(l * B * 4 * H, (B, 4 * H)), ctx.empty(B, H)
                    ctx.call("fml_lstm_cell_bwd", gates, c_prev, c_new, dh, dc, dpre, dc_prev, 0, B, H)
                    if h_prev is zero:
                        dh = None                     # the chain started from the zero context: nothing above to receive it
                    else:
                        ctx.gemm(dpre, h_prev, self.dW[i].view(0, (4 * H, H)), 4 * H, H, B, transA=True, ldc=Z, beta=1.0)
                        dh_prev = ctx.empty(B, H)
                        ctx.gemm(dpre, self.W[i].view(0, (4 * H, H)), dh_prev, B, H, 4 * H, ldb=Z)
                        dh = dh_prev
                    dc = dc_prev if l > 0 else None
                dctx = dh                             # gradient of this tier's initial hidden state = the tier above's output
                ctx.call("fml_col_sum", dpre_all, self.db[i], L * B, 4 * H, 1)
                need_rows = i > 0 or want_dx
                for bq in range(B):
                    rows = data[i].view((bq * lens[i] + first) * I, (L, I))
                    ctx.gemm(dpre_all.view(bq * 4 * H, (L, 4 * H)), rows, self.dW[i].view(H, (4 * H, I)), 4 * H, I, L, transA=True,
                             lda=B * 4 * H, ldc=Z, beta=1.0)
                    if need_rows:
                        ctx.gemm(dpre_all.view(bq * 4 * H, (L, 4 * H)), self.W[i].view(H, (4 * H, I)),
                                 grad_level(i).view((bq * lens[i] + first) * I, (L, I)), L, I, 4 * H, lda=B * 4 * H, ldb=Z, beta=1.0)
            # ---- aggregation levels, highest first: dS -> dZ = dS (1 - S^2), then into the weights and the level below
            for i in range(len(self.grainingSizes) - 1, -1, -1):
                cnt, grain = lens[i + 1], self.grainingSizes[i]
                if cnt == 0 or ddata[i + 1] is None:
                    continue
                dZ = ctx.empty(B, cnt, I)
                ctx.call("fml_act_bwd", _lib_act("tanh"), data[i + 1], ddata[i + 1], dZ, B * cnt, I, 0, self.ab[i].grad, launches=2)
                need_rows = i > 0 or want_dx
                for bq in range(B):
                    chunks = data[i].view(bq * lens[i] * I, (cnt, grain * I))
                    ctx.gemm(dZ.view(bq * cnt * I, (cnt, I)), chunks, self.aW[i].grad, I, grain * I, cnt, transA=True, beta=1.0)
                    if need_rows:
                        ctx.gemm(dZ.view(bq * cnt * I, (cnt, I)), self.aW[i].value, grad_level(i).view(bq * lens[i] * I, (cnt, grain * I)),
                                 cnt, grain * I, I, beta=1.0)
            if want_dx:
                x._add_grad(grad_level(0).view(0, x.shape), alias=False)
        out.creator = T.Node([x] + self._params, bw, self.name, cost=8 * sum(t[1] for t in tiers) * B * H * Z)
        return out


def _lib_act(name: str) -> int:
    from . import _lib
    return _lib.ACT_BY_NAME[name]


class LayerNormalization(Layer):
    """lib/transformer/layerNormalization.dart:11-44: gamma = 1, beta = 0, epsilon = 1e-5."""

    name = "layer_norm"

    def __init__(self, epsilon: float = 1e-5):
        super().__init__()
        self.epsilon = epsilon
        self.gamma = self.beta = None

    @property
    def parameters(self):
        return [self.gamma, self.beta]

    def build(self, x: Tensor):
        d = x.shape[1]
        self.gamma, self.beta = Tensor(np.ones(d, dtype=np.float32), x.ctx), Tensor(np.zeros(d, dtype=np.float32), x.ctx)
        super().build(x)

    def forward(self, x: Tensor, residual: Optional[Tensor] = None, alias_residual_grad: bool = False) -> Tensor:
        return T.layerNorm(x, self.gamma, self.beta, self.epsilon, residual, alias_residual_grad)

    def call(self, x, residual=None, alias_residual_grad=False):
        if not self._built:
            self.build(x)
        return self.forward(x, residual, alias_residual_grad)

    __call__ = call


class MultiHeadAttention(Layer):
    """numHeads heads of width dModel/numHeads followed by the output projection Wo, no biases
    (lib/transformer/multiHeadAttentionLayer.dart:24-85, heads as in
    lib/layertypes/singleHeadAttentionLayer.dart:25-90).

    The per-head Wq, Wk, Wv [dModel x dK] live side by side in ONE matrix Wqkv
    [dModel x 3*dModel] laid out [Q heads | K heads | V heads], so columns h*dK..(h+1)*dK of each
    third are exactly head h's reference matrix and X.Wqkv is a single product."""

    name = "multi_head_attention"

    def __init__(self, dModel: int, numHeads: int, seq_len: Optional[int] = None, causal: bool = False, seed: int = 0,
                 head_weights=None, Wo=None, precision: int = -1):
        """Argument order of the reference: MultiHeadAttention(dModel, numHeads) (multiHeadAttentionLayer.dart:33)."""
        super().__init__()
        if numHeads <= 0 or dModel % numHeads != 0:
            raise ValueError(f"MultiHeadAttention(dModel={dModel}, numHeads={numHeads}): dModel must be a multiple of numHeads")
        self.numHeads, self.dModel, self.dK = numHeads, dModel, dModel // numHeads
        self.seq_len, self.causal, self.seed, self.precision = seq_len, causal, seed, precision
        self._heads0, self._wo0 = head_weights, Wo
        self.Wqkv = self.Wo = None
        self.lastAttentionWeights = None

    @staticmethod
    def pack_heads(heads):
        """[(Wq,Wk,Wv)] per head -> Wqkv [dModel x 3*dModel]."""
        return np.concatenate([np.concatenate([h[i] for h in heads], axis=1) for i in range(3)], axis=1)

    @staticmethod
    def unpack_heads(wqkv, numHeads):
        d = wqkv.shape[1] // 3
        dk = d // numHeads
        return [tuple(wqkv[:, i * d + h * dk:i * d + (h + 1) * dk] for i in range(3)) for h in range(numHeads)]

    @property
    def parameters(self):
        return [self.Wqkv, self.Wo]

    def build(self, x: Tensor):
        d = self.dModel
        a = math.sqrt(1.0 / d)  # uniform(+-sqrt(1/rows)), singleHeadAttentionLayer.dart:51-56
        if self._heads0 is not None:
            wqkv = self.pack_heads(self._heads0)
        else:
            wqkv = synth.uniform(self.seed, 0, (d, 3 * d), -a, a)
        wo = self._wo0 if self._wo0 is not None else synth.uniform(self.seed, 1, (d, d), -a, a)
        self.Wqkv, self.Wo = Tensor(np.ascontiguousarray(wqkv, dtype=np.float32), x.ctx), Tensor(wo, x.ctx)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        S = self.seq_len or x.shape[0]
        n_seq = x.shape[0] // S
        qkv = T.denseMatrix(x, self.Wqkv, None, None, self.precision)
        o = T.attentionCore(qkv, n_seq, S, self.numHeads, self.dK, self.causal, self.precision)
        self.lastAttentionWeights = o.attention_weights
        return T.denseMatrix(o, self.Wo, None, None, self.precision)


class SingleHeadAttention(MultiHeadAttention):
    """lib/layertypes/singleHeadAttentionLayer.dart:25-90 (one head, no output projection)."""

    name = "single_head_attention"

    def __init__(self, dModel: int, dK: int, dV: int, seq_len=None, causal=False, seed: int = 0, weights=None, precision=-1):
        assert dK == dV == dModel, "the fused kernel path covers dK = dV = dModel for a single head"
        super().__init__(dModel, 1, seq_len, causal, seed, [weights] if weights is not None else None, None, precision)

    @property
    def parameters(self):
        return [self.Wqkv]

    def forward(self, x: Tensor) -> Tensor:
        S = self.seq_len or x.shape[0]
        qkv = T.denseMatrix(x, self.Wqkv, None, None, self.precision)
        o = T.attentionCore(qkv, x.shape[0] // S, S, 1, self.dK, self.causal, self.precision)
        self.lastAttentionWeights = o.attention_weights
        return o


class TransformerEncoderBlock(Layer):
    """Post-LN block h = LN1(x + MHA(x)), y = LN2(h + FFN(h)), FFN = Dense(dff, ReLU) -> Dense(dModel)
    (lib/transformer/transformerEncodingLayer.dart:21-71)."""

    name = "transformer_encoder_block"

    def __init__(self, dModel: int, numHeads: int, dff: int, seq_len=None, causal=False, seed: int = 0, params=None,
                 precision: int = -1):
        super().__init__()
        p = params or {}
        self.attention = MultiHeadAttention(dModel, numHeads, seq_len, causal, seed, p.get("heads"), p.get("Wo"), precision)
        self.norm1, self.norm2 = LayerNormalization(), LayerNormalization()
        self.ffn1 = DenseLayerMatrix(dff, "relu", seed + 1, p.get("W1"), p.get("b1"), precision)
        self.ffn2 = DenseLayerMatrix(dModel, None, seed + 2, p.get("W2"), p.get("b2"), precision)
        self._p0 = p

    @property
    def parameters(self):
        return (self.attention.parameters + self.norm1.parameters + self.ffn1.parameters + self.ffn2.parameters +
                self.norm2.parameters)

    def build(self, x: Tensor):
        for layer in (self.attention, self.norm1, self.norm2):
            layer.build(x)
        for name, layer in (("1", self.norm1), ("2", self.norm2)):
            if "g" + name in self._p0:
                layer.gamma = Tensor(self._p0["g" + name], x.ctx)
                layer.beta = Tensor(self._p0["be" + name], x.ctx)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        a = self.attention(x)
        h = self.norm1(x, residual=a, alias_residual_grad=True)
        f = self.ffn2(self.ffn1(h))
        return self.norm2(h, residual=f, alias_residual_grad=True)


class PositionalEncoding(Layer):
    """x + PE[0:S] (lib/transformer/positionalEncodingLayer.dart:15-66; the table keeps the reference's exponent
    2i/dModel for every column i, :41).  No parameters.  Input [S x dModel] (one sequence, the reference's form) or
    a batch flattened into rows [n_seq*S x dModel] with `seq_len=S`: the table rows repeat per sequence.  The
    embedding layer can add the same table inside its gather (`EmbeddingLayer(positional_max_len=...)`); this class
    is the stand-alone node."""

    name = "positional_encoding"

    def __init__(self, maxSequenceLength: int, dModel: int, seq_len: int = 0):
        super().__init__()
        self.maxSequenceLength, self.dModel, self.seq_len = maxSequenceLength, dModel, seq_len
        self._tiled = {}

    def build(self, x: Tensor):
        self.pe = x.ctx.empty(self.maxSequenceLength, self.dModel)
        x.ctx.call("fml_positional_table", self.pe, self.maxSequenceLength, self.dModel)
        super().build(x)

    def forward(self, x: Tensor) -> Tensor:
        rows, d = x.shape
        S = self.seq_len or rows
        if d != self.dModel or S > self.maxSequenceLength or rows % S:
            raise ValueError("PositionalEncoding: input does not fit the table")
        if rows not in self._tiled:      # the constant addend for this shape, built once on the device
            if rows == S:
                self._tiled[rows] = Tensor(self.pe.view(0, (S, d)), x.ctx)
            else:
                tiled = x.ctx.empty(rows, d)
                for q in range(rows // S):
                    x.ctx.copy(tiled.view(q * S * d, (S, d)), self.pe.view(0, (S, d)))
                self._tiled[rows] = Tensor(tiled, x.ctx)
        return T.addMatrix(x, self._tiled[rows])


class EmbeddingLayer(Layer):
    """Row gather by token id (lib/transformer/embeddingLayer.dart:18-69), init uniform(+-0.01)
    (:38).  With `positional`, the reference's PositionalEncoding table
    (lib/transformer/positionalEncodingLayer.dart:15-66) is added in the same pass."""

    name = "embedding"

    def __init__(self, vocabSize: int, embeddingDimension: int, positional_max_len: int = 0, seed: int = 0, table=None):
        super().__init__()
        self.vocabSize, self.embeddingDimension, self.seed = vocabSize, embeddingDimension, seed
        self.positional_max_len, self._t0 = positional_max_len, table
        self.embeddings = self.pe = None

    @property
    def parameters(self):
        return [self.embeddings]

    def build_on(self, ctx):
        t = self._t0 if self._t0 is not None else synth.uniform(self.seed, 0, (self.vocabSize, self.embeddingDimension), -0.01, 0.01)
        self.embeddings = Tensor(t, ctx)
        if self.positional_max_len:
            self.pe = ctx.empty(self.positional_max_len, self.embeddingDimension)
            ctx.call("fml_positional_table", self.pe, self.positional_max_len, self.embeddingDimension)
        self._built = True

    def call(self, ids, ctx=None):
        """ids: DeviceArray of int32 token ids (any shape, read flat)."""
        if not self._built:
            self.build_on(ctx or ids.ctx)
        return T.embeddingLookup(self.embeddings, ids, self.pe, self.positional_max_len)

    __call__ = call
