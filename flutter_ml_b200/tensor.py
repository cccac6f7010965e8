"""Device-resident mirror of the reference autograd core (lib/autogradEngine/tensor.dart).

`Tensor` keeps `value`, `grad` and `creator` like the reference class (tensor.dart:21-41), but
both arrays live in HBM as float32 and every op is one or a few launches of the C-ABI
kernels.  `Node` carries the same fields (`inputs`, `backwardFn`, `opName`, `cost`,
`extraParams`, tensor.dart:5-19), `backward()` walks the tape the same way
(tensor.dart:43-75), and the free functions keep the reference's names.

Gradient accumulation follows the reference (`+=` everywhere, e.g. tensor.dart:918-924) with
one optimisation: a tensor whose `grad` does not exist yet receives its first contribution by
plain write (beta = 0) instead of zero-fill + add.  Parameters keep their grads between
`backward()` calls, so per-sample passes add up exactly as on the reference.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import ACT_BY_NAME, Context, DeviceArray

_default_ctx: Optional[Context] = None

# Epilogue fusions that need global LOADS inside the GEMM epilogue are implemented and tested but off by default:
# the epilogue warps are latency-bound and each of their loads is fully exposed (measured on B200: the dX product
# with the act'() multiply 386 us against 223 us + 132 us for product + separate kernel, but then one more
# column-sum pass for the bias gradient; softmax-backward epilogue 670 us against 263 + 237 us).
FUSE_DACT_INTO_DX = False
FUSE_SOFTMAX_BACKWARD = False
FUSE_ATTENTION = True   # one kernel for softmax(scale Q.K^T).V (TF32 mode, d_head 64, seq_len % 128 == 0)
fused_attention_calls = 0   # forward passes that took the fused kernels (lets a test prove which path it compared)


def default_context() -> Context:
    """The process-wide context (device 0 unless set_default_context was called)."""
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context()
    return _default_ctx


def set_default_context(ctx: Context) -> None:
    global _default_ctx
    _default_ctx = ctx


class Node:
    """tensor.dart:5-19."""

    __slots__ = ("inputs", "backwardFn", "opName", "cost", "extraParams")

    def __init__(self, inputs, backwardFn, opName="", cost=0, extraParams=None):
        self.inputs, self.backwardFn, self.opName, self.cost = list(inputs), backwardFn, opName, cost
        self.extraParams = extraParams or {}
        for i in self.inputs:  # consumer count: a tensor used once receives its whole gradient from one node
            i._nuse = getattr(i, "_nuse", 0) + 1


class Tensor:
    """tensor.dart:21-91.  `value` is a DeviceArray; host data (lists, numpy) is uploaded."""

    def __init__(self, value, ctx: Optional[Context] = None, requires_zero_grad: bool = False):
        self.ctx = ctx or (value.ctx if isinstance(value, DeviceArray) else default_context())
        self.value: DeviceArray = value if isinstance(value, DeviceArray) else self.ctx.upload(np.asarray(value))
        self.grad: Optional[DeviceArray] = None
        self.creator: Optional[Node] = None
        if requires_zero_grad:
            self.zeroGrad()

    @property
    def shape(self):
        return self.value.shape

    def numpy(self, dtype=np.float32):
        return self.value.numpy(dtype)

    def grad_numpy(self, dtype=np.float32):
        return self.grad.numpy(dtype)

    def zeroGrad(self):
        """tensor.dart:77-91."""
        if self.grad is None:
            self.grad = self.ctx.zeros(*self.value.shape)
        else:
            self.ctx.zero(self.grad)

    # -- gradient fan-in -------------------------------------------------------------------
    def _grad_target(self):
        """(buffer, accumulate): a fresh buffer to be written, or the existing one to add into."""
        if self.grad is None:
            self.grad = self.ctx.empty(*self.value.shape)
            return self.grad, False
        return self.grad, True

    def _add_grad(self, g: DeviceArray, scale: float = 1.0, alias: bool = False):
        """grad += scale * g.  `alias=True` lets a tensor without a grad adopt `g` itself instead
        of a copy; only for callers that know no other reader of `g` runs after a later
        accumulation into this tensor."""
        if self.grad is None and scale == 1.0:
            if alias:
                self.grad = g
            else:
                self.grad = self.ctx.empty(*self.value.shape)
                self.ctx.copy(self.grad, g)
            return
        buf, acc = self._grad_target()
        if not acc:
            self.ctx.zero(buf)
        self.ctx.call("fml_axpy", float(scale), g, buf, buf.size)

    def backward(self, retain_graph: bool = False, before=None):
        """Topological order by depth-first search over creators, seed gradient 1, closures in
        reverse (tensor.dart:43-75).  Unless `retain_graph`, the creators are dropped afterwards: every
        closure refers to its own output tensor, a reference cycle that would keep the saved
        activations in device memory until Python's cycle collector happens to run."""
        topo, seen, stack = [], set(), [(self, False)]
        while stack:
            t, done = stack.pop()
            if done:
                topo.append(t)
                continue
            if id(t) in seen:
                continue
            seen.add(id(t))
            stack.append((t, True))
            if t.creator is not None:
                for i in reversed(t.creator.inputs):
                    if id(i) not in seen:
                        stack.append((i, False))
        if self.grad is None:  # seed gradient 1 (tensor.dart:70), filled on the device: no host copy, no sync
            self.grad = self.ctx.empty(*self.value.shape)
            self.ctx.call("fml_fill", self.grad, self.grad.size, 1.0)
        # `before`: {id(tensor): callable} run just before that tensor's creator, i.e. once every consumer
        # of the tensor has contributed its gradient (used to start exchanging finished gradient slices)
        for t in reversed(topo):
            if before and id(t) in before:
                before[id(t)]()
            if t.creator is not None:
                t.creator.backwardFn()
        if not retain_graph:
            for t in topo:
                t.creator = None

    def detach_graph(self):
        """Drop creators (and with them saved activations) reachable from this tensor."""
        stack = [self]
        while stack:
            t = stack.pop()
            if t.creator is not None:
                stack.extend(t.creator.inputs)
                t.creator = None


def _rows_cols(t: Tensor):
    s = t.value.shape
    return (s[0], s[1]) if len(s) == 2 else (1, s[0])


# ----------------------------------------------------------------------------- contraction


def matMul(a: Tensor, b: Tensor, precision: int = -1) -> Tensor:
    """C = A.B (tensor.dart:867-899); backward dA += dC.B^T, dB += A^T.dC (:906-942)."""
    ctx = a.ctx
    M, K = a.shape
    K2, N = b.shape
    assert K == K2, "matMul: inner dimensions differ"
    out = Tensor(ctx.empty(M, N), ctx)

    def bw():
        ga, acc_a = a._grad_target()
        ctx.gemm(out.grad, b.value, ga, M, K, N, transB=True, beta=1.0 if acc_a else 0.0, precision=precision)
        gb, acc_b = b._grad_target()
        ctx.gemm(a.value, out.grad, gb, K, N, M, transA=True, beta=1.0 if acc_b else 0.0, precision=precision)
    ctx.gemm(a.value, b.value, out.value, M, N, K, precision=precision)
    out.creator = Node([a, b], bw, "matMul", 2 * M * K * N)
    return out


def denseMatrix(x: Tensor, W: Tensor, b: Optional[Tensor], act=None, precision: int = -1) -> Tensor:
    """act(X.W + b): matMul + addMatrixAndVector + activation of DenseLayerMatrix.forward
    (lib/layertypes/denseLayer.dart:116-125) as one fused launch; one tape node instead of three."""
    ctx = x.ctx
    M, K = x.shape
    N = W.shape[1]
    code = ACT_BY_NAME[act]
    out = Tensor(ctx.empty(M, N), ctx)
    # ReLU's gate x > 0 (tensor.dart:1030) equals y > 0, so only GELU needs the pre-activation
    z = ctx.empty(M, N) if code == _lib.ACT_GELU else None
    ctx.gemm(x.value, W.value, out.value, M, N, K, bias=b.value if b is not None else None, preact=z, act=code,
             precision=precision)
    saved = z if code == _lib.ACT_GELU else out.value
    if code != _lib.ACT_NONE:
        out._dact = (code, saved)  # lets the single consumer's dX product apply act'() in its epilogue

    def bw():
        if b is not None and b.grad is None:
            b.zeroGrad()
        if code == _lib.ACT_NONE or getattr(out, "_grad_is_dz", False):
            dz = out.grad  # already dLoss/dZ (no activation, or act' applied by the consumer's product)
            if b is not None:
                pre = getattr(out, "_dbias", None)   # column sums already formed by the loss kernel
                if pre is not None:
                    ctx.call("fml_axpy", 1.0, pre, b.grad, N)
                else:
                    ctx.call("fml_col_sum", dz, b.grad, M, N, 1)
        else:
            dz = ctx.empty(M, N)
            ctx.call("fml_act_bwd", code, saved, out.grad, dz, M, N, 0, b.grad if b is not None else None,
                     launches=2 if b is not None else 1)
        gx, acc_x = x._grad_target()
        fuse = FUSE_DACT_INTO_DX and (not acc_x) and getattr(x, "_dact", None) is not None and getattr(x, "_nuse", 0) == 1
        if fuse:
            # x is the activated output of the dense layer below and nothing else consumes it: the product
            # that forms dLoss/dx multiplies by act'() on the way out (tensor.dart:1030 / :552 / :598)
            ctx.gemm(dz, W.value, gx, M, K, N, transB=True, precision=precision, dact_saved=x._dact[1], dact=x._dact[0])
            x._grad_is_dz = True
        else:
            ctx.gemm(dz, W.value, gx, M, K, N, transB=True, beta=1.0 if acc_x else 0.0, precision=precision)
        gw, acc_w = W._grad_target()
        ctx.gemm(x.value, dz, gw, K, N, M, transA=True, beta=1.0 if acc_w else 0.0, precision=precision)
    out.creator = Node([x, W] + ([b] if b is not None else []), bw, "dense_matrix", 2 * M * K * N,
                       {"act": act or "none"})
    return out


def addMatrixAndVector(m: Tensor, v: Tensor) -> Tensor:
    """tensor.dart:679-709."""
    ctx = m.ctx
    R, C = m.shape
    out = Tensor(ctx.empty(R, C), ctx)
    ctx.call("fml_add_bias", m.value, v.value, out.value, R, C)

    def bw():
        m._add_grad(out.grad)
        if v.grad is None:
            v.zeroGrad()
        ctx.call("fml_col_sum", out.grad, v.grad, R, C, 1)
    out.creator = Node([m, v], bw, "addMatrixAndVector", R * C)
    return out


def addMatrix(a: Tensor, b: Tensor) -> Tensor:
    """tensor.dart:651-677."""
    ctx = a.ctx
    out = Tensor(ctx.empty(*a.shape), ctx)
    ctx.call("fml_add", a.value, b.value, out.value, a.value.size)

    def bw():
        a._add_grad(out.grad)
        b._add_grad(out.grad)
    out.creator = Node([a, b], bw, "add_matrix", a.value.size)
    return out


addVector = addMatrix  # tensor.dart:395-414, same arithmetic on a 1-D value


def elementWiseMultiply(a: Tensor, b: Tensor) -> Tensor:
    """tensor.dart:478-497 (matrix form :838-864)."""
    ctx = a.ctx
    out = Tensor(ctx.empty(*a.shape), ctx)
    ctx.call("fml_mul", a.value, b.value, out.value, a.value.size)

    def bw():
        for t, other in ((a, b), (b, a)):
            tmp = ctx.empty(*a.shape)
            ctx.call("fml_mul", out.grad, other.value, tmp, tmp.size)
            t._add_grad(tmp)
    out.creator = Node([a, b], bw, "multiply_matrix", a.value.size)
    return out


def _activation(x: Tensor, act: str, op_name: str) -> Tensor:
    ctx = x.ctx
    code = ACT_BY_NAME[act]
    R, C = _rows_cols(x)
    out = Tensor(ctx.empty(*x.shape), ctx)
    ctx.call("fml_act_fwd", code, x.value, out.value, x.value.size)
    saved = x.value if code in (_lib.ACT_RELU, _lib.ACT_GELU) else out.value

    def bw():
        gx, acc = x._grad_target()
        ctx.call("fml_act_bwd", code, saved, out.grad, gx, R, C, 1 if acc else 0, None)
    out.creator = Node([x], bw, op_name, x.value.size)
    return out


def reluMatrix(x):      # tensor.dart:1013-1038
    return _activation(x, "relu", "relu_matrix")


def sigmoidMatrix(x):   # tensor.dart:1123-1151
    return _activation(x, "sigmoid", "sigmoid_matrix")


def tanhMatrix(x):      # tensor.dart:1178-1209
    return _activation(x, "tanh", "tanh_matrix")


def geluMatrix(x):      # extension: exact GELU
    return _activation(x, "gelu", "gelu")


def _activation2(x: Tensor, kind: int, alpha: float, op_name: str) -> Tensor:
    """Parameterised activations: forward y = f(x), backward dx += dy * f'(x) from the saved input."""
    ctx = x.ctx
    out = Tensor(ctx.empty(*x.shape), ctx)
    ctx.call("fml_act2_fwd", kind, float(alpha), x.value, out.value, x.value.size)
    saved = x.value

    def bw():
        gx, acc = x._grad_target()
        ctx.call("fml_act2_bwd", kind, float(alpha), saved, out.grad, gx, saved.size, 1 if acc else 0)
    out.creator = Node([x], bw, op_name, x.value.size)
    return out


def leakyReluMatrix(x, alpha: float = 0.01):   # lib/activationFunctions/leakyRelu.dart:35-48
    return _activation2(x, 5, alpha, "leaky_relu")


def eluMatrix(x, alpha: float = 1.0):          # lib/activationFunctions/elu.dart:27-41
    return _activation2(x, 6, alpha, "elu")


def swishMatrix(x):                            # lib/activationFunctions/silu.dart:29-49
    return _activation2(x, 7, 0.0, "swish")


def mishMatrix(x):                             # lib/activationFunctions/mish.dart:29-31
    return _activation2(x, 8, 0.0, "mish")


ACT2_BY_NAME = {"leaky_relu": leakyReluMatrix, "elu": eluMatrix, "swish": swishMatrix, "silu": swishMatrix,
                "mish": mishMatrix}

relu, sigmoid, vectorTanh = reluMatrix, sigmoidMatrix, tanhMatrix  # vector forms :521, :541, :581


def scaleMatrix(x: Tensor, s: float) -> Tensor:
    """tensor.dart:1075-1101."""
    ctx = x.ctx
    out = Tensor(ctx.zeros(*x.shape), ctx)
    ctx.call("fml_axpy", float(s), x.value, out.value, x.value.size)

    def bw():
        x._add_grad(out.grad, float(s))
    out.creator = Node([x], bw, "scale_matrix", x.value.size, {"s": s})
    return out


def transpose(x: Tensor) -> Tensor:
    """tensor.dart:1211-1236."""
    ctx = x.ctx
    R, C = x.shape
    out = Tensor(ctx.empty(C, R), ctx)
    ctx.call("fml_transpose", x.value, out.value, R, C)

    def bw():
        tmp = ctx.empty(R, C)
        ctx.call("fml_transpose", out.grad, tmp, C, R)
        x._add_grad(tmp)
    out.creator = Node([x], bw, "transpose", R * C)
    return out


def softmaxMatrix(x: Tensor, scale: float = 1.0, causal_period: int = 0) -> Tensor:
    """Row softmax (lib/activationFunctions/softmax.dart:68-115); `scale` folds the preceding
    scaleMatrix in and `causal_period` > 0 masks column j > row mod period (extension)."""
    ctx = x.ctx
    R, C = x.shape
    out = Tensor(ctx.empty(R, C), ctx)
    ctx.call("fml_softmax_rows_fwd", x.value, out.value, R, C, float(scale), int(causal_period))

    def bw():
        gx, acc = x._grad_target()
        ctx.call("fml_softmax_rows_bwd", out.value, out.grad, gx, R, C, float(scale), 1 if acc else 0)
    out.creator = Node([x], bw, "softmax_matrix", R * C * C)
    return out


def layerNorm(x: Tensor, gamma: Tensor, beta: Tensor, epsilon: float = 1e-5, residual: Optional[Tensor] = None,
              alias_residual_grad: bool = False) -> Tensor:
    """gamma * xhat + beta per row (lib/transformer/layerNormalization.dart:137-202).  With
    `residual`, normalises x + residual: the addMatrix of transformerEncodingLayer.dart:63,68 is
    read inside the same kernel instead of being written out first."""
    ctx = x.ctx
    R, C = x.shape
    out = Tensor(ctx.empty(R, C), ctx)
    xhat, rstd = ctx.empty(R, C), ctx.empty(R)
    ctx.call("fml_layernorm_fwd", x.value, residual.value if residual is not None else None, gamma.value, beta.value,
             out.value, xhat, rstd, R, C, float(epsilon))

    def bw():
        for p in (gamma, beta):
            if p.grad is None:
                p.zeroGrad()
        if residual is None:
            gx, acc = x._grad_target()
            ctx.call("fml_layernorm_bwd", out.grad, gamma.value, xhat, rstd, gx, gamma.grad, beta.grad, R, C, 1 if acc else 0)
        else:
            d = ctx.empty(R, C)
            ctx.call("fml_layernorm_bwd", out.grad, gamma.value, xhat, rstd, d, gamma.grad, beta.grad, R, C, 0)
            x._add_grad(d, alias=alias_residual_grad)
            residual._add_grad(d, alias=alias_residual_grad)
    out.creator = Node([x, gamma, beta] + ([residual] if residual is not None else []), bw, "layer_norm", R * C * 8)
    return out


def _attentionFused(qkv: Tensor, q, k, v, Bn, S, H, dk, causal, scale):
    """fml_attention_fwd / fml_attention_bwd: the score matrices stay on chip in the forward pass; the backward
    pass rebuilds the probabilities from the saved row statistics and writes only P and dS once."""
    import ctypes
    ctx = qkv.ctx
    d = H * dk
    out = Tensor(ctx.empty(Bn * S, d), ctx)
    lse = ctx.empty(Bn * H * S)
    desc = _lib.AttentionDesc()
    desc.n_seq, desc.seq_len, desc.heads, desc.d_head = Bn, S, H, dk
    desc.q, desc.k, desc.v, desc.ld_qkv = q.ptr, k.ptr, v.ptr, 3 * d
    desc.out, desc.ld_out, desc.lse = out.value.ptr, d, lse.ptr
    desc.scale, desc.causal = scale, int(bool(causal))
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, ctypes.byref(desc)))
    ctx.launches += 1
    global fused_attention_calls
    fused_attention_calls += 1

    def bw():
        g, acc = qkv._grad_target()
        scratch = ctx.empty(Bn * H * S)
        ctx.check(ctx.lib.fml_attention_bwd(ctx.h, ctypes.byref(desc), out.grad.ptr, d, g.ptr, g.ptr + 4 * d, g.ptr + 8 * d, 3 * d,
                                            1 if acc else 0, scratch.ptr))
        ctx.launches += 4
        _keep = (lse, out)  # the descriptor holds raw pointers into these
    out.creator = Node([qkv], bw, "attention", 4 * Bn * H * S * S * dk, {"causal": causal, "fused": True})
    out.attention_weights = None   # never materialised on this path (set FUSE_ATTENTION = False to inspect them)
    return out


def attentionCore(qkv: Tensor, n_seq: int, seq_len: int, heads: int, d_head: int, causal: bool, precision: int = -1):
    """Scaled dot-product attention for all (sequence, head) pairs at once, reading Q, K, V as
    column slices of the fused projection [n_seq*seq_len, 3*heads*d_head] and writing the heads
    side by side: transpose + matMul + scaleMatrix + softmaxMatrix + matMul of
    lib/layertypes/singleHeadAttentionLayer.dart:77-86 and the column concat of
    lib/transformer/multiHeadAttentionLayer.dart:80, without any of those copies."""
    ctx = qkv.ctx
    Bn, S, H, dk = n_seq, seq_len, heads, d_head
    d = H * dk
    ld = 3 * d
    scale = 1.0 / math.sqrt(dk)
    q, k, v = qkv.value, qkv.value.view(d, ()), qkv.value.view(2 * d, ())
    eff_prec = ctx.precision if precision < 0 else precision
    if FUSE_ATTENTION and eff_prec == _lib.PREC_TF32 and dk == 64 and S % 128 == 0:
        return _attentionFused(qkv, q, k, v, Bn, S, H, dk, causal, scale)
    P = ctx.empty(Bn * H * S, S)
    out = Tensor(ctx.empty(Bn * S, d), ctx)
    bat = dict(batch=(H, Bn), precision=precision)
    s_qkv, s_p, s_o = (dk, S * ld), (S * S, H * S * S), (dk, S * d)
    eff_prec = ctx.precision if precision < 0 else precision
    # scores of up to 512 keys fit one CTA's tensor memory: scale, mask and softmax run in the epilogue of the
    # Q.K^T product (and the softmax backward in the epilogue of dO.V^T), so S never makes a round trip
    fused_rows = S <= 512 and S % 32 == 0 and eff_prec != _lib.PREC_FP32
    if fused_rows:
        ctx.gemm(q, k, P, S, S, dk, transB=True, lda=ld, ldb=ld, ldc=S, sA=s_qkv, sB=s_qkv, sC=s_p, alpha=scale,
                 rowop=1, rowop_causal=causal, **bat)
    else:
        ctx.gemm(q, k, P, S, S, dk, transB=True, lda=ld, ldb=ld, ldc=S, sA=s_qkv, sB=s_qkv, sC=s_p, **bat)
        ctx.call("fml_softmax_rows_fwd", P, P, Bn * H * S, S, scale, S if causal else 0)
    ctx.gemm(P, v, out.value, S, dk, S, lda=S, ldb=ld, ldc=d, sA=s_p, sB=s_qkv, sC=s_o, **bat)

    def bw():
        g, acc = qkv._grad_target()
        if not acc:
            pass  # every element of the buffer is written below (dQ, dK, dV cover all 3*d columns)
        beta = 1.0 if acc else 0.0
        gq, gk, gv = g, g.view(d, ()), g.view(2 * d, ())
        dO = out.grad
        dP = ctx.empty(Bn * H * S, S)
        # dP = dO_h . V_h^T ; dV_h = P^T . dO_h
        # The backward row epilogue (rowop 2) exists and is tested, but re-reading P from the epilogue warps made
        # it slower than the separate kernels (670 us against 263 + 237 us per layer at 16 heads x 32 x 512^2).
        if fused_rows and FUSE_SOFTMAX_BACKWARD:
            # dS = scale * P * (dP - sum(dP*P)) straight out of the product's epilogue
            ctx.gemm(dO, v, dP, S, S, dk, transB=True, lda=d, ldb=ld, ldc=S, sA=s_o, sB=s_qkv, sC=s_p, alpha=scale,
                     rowop=2, rowop_aux=P, **bat)
        else:
            ctx.gemm(dO, v, dP, S, S, dk, transB=True, lda=d, ldb=ld, ldc=S, sA=s_o, sB=s_qkv, sC=s_p, **bat)
        ctx.gemm(P, dO, gv, S, dk, S, transA=True, lda=S, ldb=d, ldc=ld, sA=s_p, sB=s_o, sC=s_qkv, beta=beta, **bat)
        if not (fused_rows and FUSE_SOFTMAX_BACKWARD):
            # dS = scale * P * (dP - sum(dP*P)), in place over dP
            ctx.call("fml_softmax_rows_bwd", P, dP, dP, Bn * H * S, S, scale, 0)
        # dQ_h = dS . K_h ; dK_h = dS^T . Q_h
        ctx.gemm(dP, k, gq, S, dk, S, lda=S, ldb=ld, ldc=ld, sA=s_p, sB=s_qkv, sC=s_qkv, beta=beta, **bat)
        ctx.gemm(dP, q, gk, S, dk, S, transA=True, lda=S, ldb=ld, ldc=ld, sA=s_p, sB=s_qkv, sC=s_qkv, beta=beta, **bat)
    out.creator = Node([qkv], bw, "attention", 4 * Bn * H * S * S * dk, {"causal": causal})
    out.attention_weights = P
    return out


def conv2dBatch(x: Tensor, kernels: Tensor, biases: Optional[Tensor], kh: int, kw: int, padding: str = "valid") -> Tensor:
    """conv2d (tensor.dart:765-833) of every image in x [n_img, H, W] with every kernel in `kernels`
    [n_k, kh*kw] (x may also be one matrix [H, W]), plus addScalarToMatrix of `biases` [n_k] (tensor.dart:711-737): Conv2DLayer.forward
    (lib/layertypes/conv2d.dart:60-75) as one launch.  Output [n_img, n_k, OH, OW]."""
    ctx = x.ctx
    single = len(x.shape) == 2   # one matrix, as in the reference
    n_img, H, W = (1,) + tuple(x.shape) if single else x.shape
    n_k = kernels.shape[0]
    pad = (kh - 1) // 2 if padding == "same" else 0
    OH, OW = H + 2 * pad - kh + 1, W + 2 * pad - kw + 1
    out = Tensor(ctx.empty(*((n_k, OH, OW) if single else (n_img, n_k, OH, OW))), ctx)
    args = (n_img, H, W, n_k, kh, kw, pad)
    ctx.call("fml_conv2d_fwd", x.value, kernels.value, biases.value if biases is not None else None, out.value, *args)

    def bw():
        for t in (x, kernels, biases):
            if t is not None and t.grad is None:
                t.zeroGrad()   # the backward kernels add into their targets
        ctx.call("fml_conv2d_bwd", x.value, kernels.value, out.grad, x.grad, kernels.grad,
                 biases.grad if biases is not None else None, *args, launches=2)
    out.creator = Node([x, kernels] + ([biases] if biases is not None else []), bw, "conv2d", 2 * n_img * n_k * OH * OW * kh * kw,
                       {"padding": padding})
    return out


# --------------------------------------------------------------------------------- losses


def mseMatrix(pred: Tensor, target: Tensor, weight: float = 1.0) -> Tensor:
    """mean((p-t)^2) * weight (tensor.dart:982-1011; vector form mse :499-519).  The gradient
    2(p-t)/n * weight is produced by the same pass."""
    ctx = pred.ctx
    n = pred.value.size
    out = Tensor(ctx.zeros(1), ctx)
    dp = ctx.empty(*pred.shape)
    ctx.call("fml_mse", pred.value, target.value, dp, out.value, n, 1.0, launches=2)
    if weight != 1.0:
        tmp = ctx.zeros(1)
        ctx.call("fml_axpy", float(weight), out.value, tmp, 1)
        out.value = tmp

    def bw():
        pred._add_grad(dp, float(weight))
    out.creator = Node([pred], bw, "mse_matrix", 3 * n)
    return out


mse = mseMatrix


def softmaxCrossEntropy(logits: Tensor, labels: DeviceArray, inv_count: float, bias_grad: bool = False) -> Tensor:
    """Extension (the reference has only mse / binaryCrossEntropy): sum over rows of
    -log softmax(z)[label] * inv_count.  The gradient overwrites the logits buffer in the same
    kernel, so the [tokens x vocab] tensor exists once.  With `bias_grad` the same kernel also sums the
    gradient over the rows; the dense node that produced the logits then adds that vector to its bias
    gradient instead of reading the [tokens x vocab] gradient again (tensor.dart:698-704)."""
    ctx = logits.ctx
    R, C = logits.shape
    out = Tensor(ctx.zeros(1), ctx)
    if bias_grad:
        db = ctx.zeros(C)
        ctx.call("fml_softmax_xent_dbias", logits.value, labels, logits.value, out.value, R, C, float(inv_count), db, launches=3)
        logits._dbias = db
    else:
        ctx.call("fml_softmax_xent", logits.value, labels, logits.value, out.value, R, C, float(inv_count), launches=2)

    def bw():
        logits._add_grad(logits.value, alias=True)
    out.creator = Node([logits], bw, "softmax_xent", 4 * R * C)
    return out


def embeddingLookup(table: Tensor, ids: DeviceArray, pe: Optional[DeviceArray] = None, period: int = 0) -> Tensor:
    """Row gather (lib/transformer/embeddingLayer.dart:47-56) with the positional table added in
    the same pass (positionalEncodingLayer.dart:55-65); backward scatter-adds (:58-65)."""
    ctx = table.ctx
    n, dim = ids.size, table.shape[1]
    out = Tensor(ctx.empty(n, dim), ctx)
    ctx.call("fml_embedding_fwd", table.value, ids, pe, out.value, n, dim, int(period), table.shape[0])

    def bw():
        if table.grad is None:
            table.zeroGrad()
        ctx.call("fml_embedding_bwd", out.grad, ids, table.grad, n, dim, table.shape[0])
    out.creator = Node([table], bw, "embedding_lookup", 0)
    return out


def concatenateMatricesByColumn(parts: Sequence[Tensor]) -> Tensor:
    """tensor.dart:739-763.  Kept for API parity; the attention path writes heads side by side
    directly and never calls it."""
    ctx = parts[0].ctx
    host = np.concatenate([p.numpy() for p in parts], axis=1)
    out = Tensor(ctx.upload(host), ctx)

    def bw():
        g = out.grad.numpy()
        c = 0
        for p in parts:
            w = p.shape[1]
            p._add_grad(ctx.upload(np.ascontiguousarray(g[:, c:c + w])))
            c += w
    out.creator = Node(list(parts), bw, "concat_matrix_col", 0)
    return out
