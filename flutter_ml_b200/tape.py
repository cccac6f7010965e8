"""Host side of the tape executor: records autograd nodes under the reference's function names and
runs the whole list with ONE library call per sweep (`fml_tape_run`).

The reference walks `Node.inputs / opName / extraParams` (lib/autogradEngine/tensor.dart:5-19) and
calls one closure per node (`Tensor.backward`, tensor.dart:43-75).  A Dart executor over the C ABI
does what `Tape` does here: while the model's forward code runs it appends one `fml_op` per node
(device buffers for value and gradient instead of nested lists), then `forward()` / `backward()`
submit the list.  Gradients accumulate (+=) into leaf tensors until `zeroGrad`, as in the
reference; gradients of intermediate tensors live in one arena that `backward()` clears with a
single memset first (every reference forward pass creates fresh tensors with zero gradients,
tensor.dart:26-41).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _lib

KIND = {"matMul": 1, "matVecMul": 2, "addMatrixAndVector": 3, "add": 4, "multiply": 5, "relu": 6, "sigmoid": 7,
        "tanh": 8, "gelu": 9, "leaky_relu": 10, "elu": 11, "swish": 12, "mish": 13, "scale_matrix": 14,
        "transpose": 15, "concat": 16, "softmax_matrix": 17, "layer_norm": 18, "embedding_lookup": 19, "mse": 20,
        "sum": 21, "softmax_xent": 22, "dense": 23, "conv2d": 24, "addScalarToMatrix": 25, "attention": 26}
FORWARD, BACKWARD, BACKWARD_NOSEED = 0, 1, 2


class TapeTensor:
    """rows x cols floats on the device; `grad` has the same shape (None until someone needs it)."""

    def __init__(self, tape, rows, cols, value=None, grad=None, leaf=False):
        self.tape, self.rows, self.cols, self.value, self.grad, self.leaf = tape, rows, cols, value, grad, leaf

    @property
    def shape(self):
        return (self.rows, self.cols)

    def numpy(self, dtype=np.float32):
        return self.value.numpy(dtype).reshape(self.rows, self.cols)

    def grad_numpy(self, dtype=np.float32):
        return self.grad.numpy(dtype).reshape(self.rows, self.cols)

    def zeroGrad(self):
        """Tensor.zeroGrad (tensor.dart:77-91)."""
        if self.grad is not None:
            self.tape.ctx.zero(self.grad)


class Tape:
    def __init__(self, ctx: _lib.Context, precision: int = -1):
        self.ctx, self.precision = ctx, precision
        self._recs: List[dict] = []       # recorded nodes, in creation order
        self._inter: List[TapeTensor] = []  # tensors created by nodes
        self._ops = None
        self._keep = []                   # host arrays and device buffers the op list points into

    # ------------------------------------------------------------------ tensors
    def tensor(self, value, requires_grad: bool = True) -> TapeTensor:
        """A leaf: parameters and inputs (vectors become 1 x n)."""
        a = np.asarray(value, dtype=np.float32)
        a = a.reshape(1, -1) if a.ndim <= 1 else a
        t = TapeTensor(self, a.shape[0], a.shape[1], self.ctx.upload(a), leaf=True)
        if requires_grad:
            t.grad = self.ctx.zeros(*a.shape)
        return t

    def ids(self, values):
        return self.ctx.upload(np.asarray(values, dtype=np.int32).ravel())

    def _new(self, rows, cols) -> TapeTensor:
        t = TapeTensor(self, rows, cols)
        self._inter.append(t)
        return t

    def _record(self, kind, out, ins=(), inner=0, aux=(), ids=None, parts=None, s=0.0, iparam=0):
        assert self._ops is None, "the tape is compiled; record a new Tape for a different graph"
        self._recs.append(dict(kind=KIND[kind], out=out, ins=list(ins), inner=inner, aux=list(aux), ids=ids,
                               parts=parts, s=float(s), iparam=int(iparam)))
        return out

    # ------------------------------------------------------------------ the reference's functions
    def matMul(self, a, b):                       # tensor.dart:867-947
        assert a.cols == b.rows
        return self._record("matMul", self._new(a.rows, b.cols), (a, b), inner=a.cols)

    def matVecMul(self, M, v):                    # tensor.dart:949-980
        assert v.rows == 1 and M.cols == v.cols
        return self._record("matVecMul", self._new(1, M.rows), (M, v), inner=M.cols)

    def addMatrixAndVector(self, m, v):           # tensor.dart:679-709
        assert v.rows == 1 and v.cols == m.cols
        return self._record("addMatrixAndVector", self._new(m.rows, m.cols), (m, v))

    def addMatrix(self, a, b):                    # tensor.dart:651-677 (addVector :395-414)
        assert a.shape == b.shape
        return self._record("add", self._new(a.rows, a.cols), (a, b))

    addVector = addMatrix

    def elementWiseMultiply(self, a, b):          # tensor.dart:478-497, 835-865
        assert a.shape == b.shape
        return self._record("multiply", self._new(a.rows, a.cols), (a, b))

    def _unary(self, kind, x, s=0.0):
        return self._record(kind, self._new(x.rows, x.cols), (x,), s=s)

    def reluMatrix(self, x):                      # tensor.dart:1013-1038 (relu :521-539)
        return self._unary("relu", x)

    def sigmoidMatrix(self, x):                   # tensor.dart:1123-1151 (sigmoid :541-559)
        return self._unary("sigmoid", x)

    def tanhMatrix(self, x):                      # tensor.dart:1178-1209 (vectorTanh :581-605)
        return self._unary("tanh", x)

    relu, sigmoid, vectorTanh = reluMatrix, sigmoidMatrix, tanhMatrix

    def gelu(self, x):                            # extension
        return self._unary("gelu", x)

    def leakyRelu(self, x, alpha=0.01):           # lib/activationFunctions/leakyRelu.dart:35-48
        return self._unary("leaky_relu", x, alpha)

    def elu(self, x, alpha=1.0):                  # lib/activationFunctions/elu.dart:27-41
        return self._unary("elu", x, alpha)

    def swish(self, x):                           # lib/activationFunctions/silu.dart:29-49
        return self._unary("swish", x)

    def mish(self, x):                            # lib/activationFunctions/mish.dart:29-31
        return self._unary("mish", x)

    def scaleMatrix(self, x, s):                  # tensor.dart:1075-1101, extraParams {'s': s}
        return self._unary("scale_matrix", x, s)

    def transpose(self, x):                       # tensor.dart:1211-1236
        return self._record("transpose", self._new(x.cols, x.rows), (x,))

    def concatenateMatricesByColumn(self, parts: Sequence[TapeTensor]):   # tensor.dart:739-763
        rows = parts[0].rows
        assert all(p.rows == rows for p in parts)
        return self._record("concat", self._new(rows, sum(p.cols for p in parts)), parts=list(parts))

    def concatenate(self, a, b):                  # tensor.dart:437-455
        return self.concatenateMatricesByColumn([a, b])

    def softmaxMatrix(self, x, causal_period: int = 0):   # lib/activationFunctions/softmax.dart:68-115
        return self._record("softmax_matrix", self._new(x.rows, x.cols), (x,), iparam=causal_period)

    def layerNorm(self, x, gamma, beta, epsilon=1e-5):    # lib/transformer/layerNormalization.dart:137-202
        aux = (self.ctx.empty(x.rows, x.cols), self.ctx.empty(x.rows))
        return self._record("layer_norm", self._new(x.rows, x.cols), (x, gamma, beta), aux=aux, s=epsilon)

    def embeddingLookup(self, table, ids):        # lib/transformer/embeddingLayer.dart:47-67
        return self._record("embedding_lookup", self._new(ids.size, table.cols), (table,), inner=table.rows, ids=ids)

    def mseMatrix(self, p, t):                    # tensor.dart:982-1011 (mse :499-519)
        assert p.shape == t.shape
        return self._record("mse", self._new(1, 1), (p, t), inner=p.rows * p.cols)

    mse = mseMatrix

    def sumMatrix(self, x):                       # tensor.dart:1153-1176 (sum :561-579)
        return self._record("sum", self._new(1, 1), (x,), inner=x.rows * x.cols)

    sum = sumMatrix

    def conv2d(self, x, kernel, padding: str = "valid"):   # tensor.dart:765-833, extraParams {'padding': ...}
        pad = (kernel.rows - 1) // 2 if padding == "same" else 0
        out = self._new(x.rows + 2 * pad - kernel.rows + 1, x.cols + 2 * pad - kernel.cols + 1)
        return self._record("conv2d", out, (x, kernel), inner=kernel.rows, iparam=kernel.cols, s=pad)

    def addScalarToMatrix(self, m, s):            # tensor.dart:711-737 (s is a 1 x 1 tensor)
        assert s.shape == (1, 1)
        return self._record("addScalarToMatrix", self._new(m.rows, m.cols), (m, s))

    def attention(self, q, k, v, seq_len: int, scale: float, causal: bool = False):   # extension: one fused node
        """softmax(scale Q.K^T [+ causal mask]) . V for rows / seq_len sequences and cols / 64 heads
        (singleHeadAttentionLayer.dart:77-86 + the head concat of multiHeadAttentionLayer.dart:80)."""
        assert q.shape == k.shape == v.shape and q.rows % seq_len == 0 and q.cols % 64 == 0
        n = q.rows * (q.cols // 64)
        aux = (self.ctx.empty(n), self.ctx.empty(n))
        return self._record("attention", self._new(q.rows, q.cols), (q, k, v), inner=seq_len, aux=aux, s=scale, iparam=int(causal))

    def softmaxCrossEntropy(self, logits, labels, inv_count):   # extension
        aux = (self.ctx.empty(logits.rows, logits.cols),)
        return self._record("softmax_xent", self._new(1, 1), (logits,), inner=logits.rows, aux=aux, ids=labels,
                            s=inv_count, iparam=logits.cols)

    def dense(self, x, W, b: Optional[TapeTensor], act=None):   # denseLayer.dart:116-125 as one node
        code = _lib.ACT_BY_NAME[act]
        aux = (self.ctx.empty(x.rows, W.cols),) if code == _lib.ACT_GELU else ()
        ins = (x, W) + ((b,) if b is not None else ())
        return self._record("dense", self._new(x.rows, W.cols), ins, inner=x.cols, aux=aux, iparam=code)

    # ------------------------------------------------------------------ compile and run
    def compile(self):
        """Allocate intermediate values and gradients (one arena each) and build the fml_op array."""
        if self._ops is not None:
            return
        ctx = self.ctx
        offs, total = [], 0
        for t in self._inter:
            offs.append(total)
            total += (t.rows * t.cols + 3) & ~3
        self._values, self._grads = ctx.empty(max(total, 4)), ctx.zeros(max(total, 4))
        for t, o in zip(self._inter, offs):
            t.value, t.grad = self._values.view(o, t.shape), self._grads.view(o, t.shape)
        ops = (_lib.Op * max(len(self._recs), 1))()
        for op, r in zip(ops, self._recs):
            out = r["out"]
            op.kind, op.rows, op.cols, op.inner = r["kind"], out.rows, out.cols, r["inner"]
            op.out, op.gout = out.value.ptr, out.grad.ptr
            for i, t in enumerate(r["ins"]):
                op.inp[i] = t.value.ptr
                op.gin[i] = t.grad.ptr if t.grad is not None else None
            for i, a in enumerate(r["aux"]):
                op.aux[i] = a.ptr
            if r["ids"] is not None:
                op.ids = r["ids"].ptr
            if r["parts"] is not None:
                ps = r["parts"]
                pv = (_lib.fp * len(ps))(*[p.value.ptr for p in ps])
                pg = (_lib.fp * len(ps))(*[p.grad.ptr if p.grad is not None else None for p in ps])
                pc = (_lib.i32 * len(ps))(*[p.cols for p in ps])
                self._keep += [pv, pg, pc]
                op.parts, op.gparts, op.part_cols, op.n_parts = (C.cast(pv, _lib.fp), C.cast(pg, _lib.fp),
                                                                 C.cast(pc, _lib.fp), len(ps))
            op.s, op.iparam, op.precision = r["s"], r["iparam"], self.precision
        self._ops = ops

    def forward(self):
        self.compile()
        self.ctx.check(self.ctx.lib.fml_tape_run(self.ctx.h, self._ops, len(self._recs), FORWARD))

    def backward(self, seed: bool = True):
        """Tensor.backward (tensor.dart:43-75) of the last recorded tensor."""
        self.compile()
        self.ctx.zero(self._grads)
        self.ctx.check(self.ctx.lib.fml_tape_run(self.ctx.h, self._ops, len(self._recs), BACKWARD if seed else BACKWARD_NOSEED))

    def __len__(self):
        return len(self._recs)
