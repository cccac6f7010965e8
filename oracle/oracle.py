"""CPU oracle bindings and reference-shaped compositions.  TEST INFRASTRUCTURE ONLY.

Loads ``oracle/liboracle.so`` (the float64 C restatement of the reference's
pure-Dart eager engine, see ``oracle.c``) and stacks its ops the way the
reference's layers do, on a tape that mirrors ``Tensor``/``Node``/``backward``
(lib/autogradEngine/tensor.dart:5-75).  Nothing in the product package imports
this module; only tests, the smoke check and the benchmark's CPU-baseline leg do.

Parity status: pinned for matMul forward by the reference's all-ones check
(lib/gpu_benching.dart:34-37,60); otherwise PARITY UNPINNED (the reference has no
golden vectors and cannot be executed here), guarded by an independent
torch-float64 autograd model and finite differences in the test-suite.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {}

_dp = C.POINTER(C.c_double)


def _p(a):
    if a is None:
        return None
    assert a.dtype == np.float64 and a.flags.c_contiguous
    return a.ctypes.data_as(_dp)


def build():
    """Compile both oracle variants with the committed Makefile."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


def lib(omp: bool = False):
    key = "omp" if omp else "st"
    if key not in _LIBS:
        path = os.path.join(_HERE, "liboracle_omp.so" if omp else "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_mse_fwd.restype = C.c_double
        L.orc_softmax_xent.restype = C.c_double
        L.orc_threads.restype = C.c_int
        _LIBS[key] = L
    return _LIBS[key]


class Ops:
    """numpy-facing wrappers around the C functions (float64, row-major)."""

    def __init__(self, omp: bool = False):
        self.L = lib(omp)

    def threads(self):
        return int(self.L.orc_threads())

    def set_threads(self, n):
        self.L.orc_set_threads(int(n))

    def matmul_fwd(self, A, B):
        M, N = A.shape
        P = B.shape[1]
        out = np.empty((M, P))
        self.L.orc_matmul_fwd(_p(A), _p(B), _p(out), M, N, P)
        return out

    def matmul_bwd(self, A, B, dC, dA, dB):
        M, N = A.shape
        P = B.shape[1]
        self.L.orc_matmul_bwd(_p(A), _p(B), _p(dC), _p(dA), _p(dB), M, N, P)

    def matvec_fwd(self, Mx, v):
        y = np.empty(Mx.shape[0])
        self.L.orc_matvec_fwd(_p(Mx), _p(v), _p(y), Mx.shape[0], Mx.shape[1])
        return y

    def matvec_bwd(self, Mx, v, dy, dM, dv):
        self.L.orc_matvec_bwd(_p(Mx), _p(v), _p(dy), _p(dM), _p(dv), Mx.shape[0], Mx.shape[1])

    def unary_fwd(self, name, x):
        y = np.empty_like(x)
        getattr(self.L, f"orc_{name}_fwd")(_p(x), _p(y), C.c_int64(x.size))
        return y

    def unary_bwd(self, name, saved, dy, dx):
        getattr(self.L, f"orc_{name}_bwd")(_p(saved), _p(dy), _p(dx), C.c_int64(dy.size))

    def softmax_fwd(self, x, causal_period=0):
        y = np.empty_like(x)
        self.L.orc_softmax_rows_fwd(_p(x), _p(y), x.shape[0], x.shape[1], causal_period)
        return y

    def softmax_bwd(self, y, dy, dx):
        self.L.orc_softmax_rows_bwd(_p(y), _p(dy), _p(dx), y.shape[0], y.shape[1])

    def layernorm_fwd(self, x, gamma, beta, eps=1e-5):
        y = np.empty_like(x)
        xhat = np.empty_like(x)
        var = np.empty(x.shape[0])
        self.L.orc_layernorm_fwd(_p(x), _p(gamma), _p(beta), _p(y), _p(xhat), _p(var),
                                 x.shape[0], x.shape[1], C.c_double(eps))
        return y, xhat, var

    def layernorm_bwd(self, dy, gamma, xhat, var, dx, dgamma, dbeta, eps=1e-5):
        self.L.orc_layernorm_bwd(_p(dy), _p(gamma), _p(xhat), _p(var), _p(dx), _p(dgamma),
                                 _p(dbeta), dy.shape[0], dy.shape[1], C.c_double(eps))

    def mse_fwd(self, p, t):
        return float(self.L.orc_mse_fwd(_p(p), _p(t), C.c_int64(p.size)))

    def mse_bwd(self, p, t, dp, upstream=1.0):
        self.L.orc_mse_bwd(_p(p), _p(t), _p(dp), C.c_int64(p.size), C.c_double(upstream))

    def softmax_xent(self, z, labels, dz, inv_count):
        labels = np.ascontiguousarray(labels, dtype=np.int32)
        return float(self.L.orc_softmax_xent(_p(z), labels.ctypes.data_as(C.POINTER(C.c_int32)),
                                             _p(dz), z.shape[0], z.shape[1], C.c_double(inv_count)))

    def sgd_step(self, w, g, lr):
        self.L.orc_sgd_step(_p(w), _p(g), C.c_int64(w.size), C.c_double(lr))

    def adam_step(self, w, g, m, v, lr, t, b1=0.9, b2=0.999, eps=1e-8):
        self.L.orc_adam_step(_p(w), _p(g), _p(m), _p(v), C.c_int64(w.size), C.c_double(lr),
                             C.c_double(b1), C.c_double(b2), C.c_double(eps), int(t))

    def optimizer_step(self, kind, w, g, s1, s2, s3, lr, h=(0, 0, 0, 0), t=1):
        """kind: 1 Momentum, 2 NAG, 3 RMSprop, 4 Adagrad, 6 AdamW, 7 AMSGrad (see oracle.c)."""
        h = list(h) + [0.0] * (4 - len(h))
        self.L.orc_optimizer_step(int(kind), _p(w), _p(g), _p(s1), _p(s2), _p(s3), C.c_int64(w.size), C.c_double(lr),
                                  *[C.c_double(x) for x in h], int(t))

    def act2_fwd(self, kind, alpha, x):
        y = np.empty_like(x)
        self.L.orc_act2_fwd(int(kind), C.c_double(alpha), _p(x), _p(y), C.c_int64(x.size))
        return y

    def act2_bwd(self, kind, alpha, x, dy, dx):
        self.L.orc_act2_bwd(int(kind), C.c_double(alpha), _p(x), _p(dy), _p(dx), C.c_int64(x.size))

    def conv2d_fwd(self, x, k, pad):
        H, W = x.shape
        kh, kw = k.shape
        out = np.empty((H + 2 * pad - kh + 1, W + 2 * pad - kw + 1))
        self.L.orc_conv2d_fwd(_p(x), _p(k), _p(out), H, W, kh, kw, pad)
        return out

    def conv2d_bwd(self, x, k, dout, dx, dk, pad):
        self.L.orc_conv2d_bwd(_p(x), _p(k), _p(dout), _p(dx), _p(dk), x.shape[0], x.shape[1], k.shape[0], k.shape[1], pad)

    def embedding_fwd(self, table, ids):
        ids = np.ascontiguousarray(ids, dtype=np.float64)
        out = np.empty((ids.size, table.shape[1]))
        self.L.orc_embedding_fwd(_p(table), _p(ids), _p(out), ids.size, table.shape[1])
        return out

    def embedding_bwd(self, dout, ids, dtable):
        ids = np.ascontiguousarray(ids, dtype=np.float64)
        self.L.orc_embedding_bwd(_p(dout), _p(ids), _p(dtable), ids.size, dtable.shape[1])

    def positional_table(self, max_len, d_model):
        pe = np.empty((max_len, d_model))
        self.L.orc_positional_table(_p(pe), max_len, d_model)
        return pe

    def lstm_fwd_bwd(self, W, b, x, target, backward=True):
        """W [4,H,H+I] (f,i,c~,o; columns [h|x]), b [4,H], x [B,T,I], target [B,H]."""
        B, T, I = x.shape
        H = W.shape[1]
        h_last = np.empty((B, H))
        loss = C.c_double(0)
        dW = np.zeros_like(W)
        db = np.zeros_like(b)
        self.L.orc_lstm_fwd_bwd(_p(W), _p(b), _p(x), _p(target), _p(h_last), C.byref(loss),
                                _p(dW), _p(db), B, T, I, H, 1 if backward else 0)
        return h_last, loss.value, dW, db


# --------------------------------------------------------------------------- tape


class T:
    """Mirror of the reference Tensor: value, zero-initialised grad, creator node
    (lib/autogradEngine/tensor.dart:21-41)."""

    def __init__(self, value):
        self.value = np.array(value, dtype=np.float64, order="C")
        self.grad = np.zeros_like(self.value)
        self.inputs = ()
        self.backward_fn = None

    def backward(self):
        """Depth-first topological sort over creators, seed gradient 1.0, closures in
        reverse order (tensor.dart:43-75)."""
        topo, seen = [], set()
        stack = [(self, False)]
        while stack:  # iterative form of the recursive visit at :54-66
            node, done = stack.pop()
            if done:
                topo.append(node)
                continue
            if id(node) in seen:
                continue
            seen.add(id(node))
            stack.append((node, True))
            for i in reversed(node.inputs):
                if id(i) not in seen:
                    stack.append((i, False))
        self.grad = np.ones_like(self.value)
        for node in reversed(topo):
            if node.backward_fn is not None:
                node.backward_fn()


def _node(out, inputs, fn):
    out.inputs = tuple(inputs)
    out.backward_fn = fn
    return out


class Engine:
    """Reference ops on the tape; each method follows the cited reference function."""

    def __init__(self, omp: bool = False):
        self.ops = Ops(omp)
        # Test aid, not reference behaviour: an iterator of boolean masks.  While it is set, every reluMatrix call
        # takes its gate pattern from the next mask instead of from the sign of its own input.  ReLU's gate is
        # discontinuous, so a device pre-activation that differs from the float64 one in the last TF32 bit can
        # land on the other side of zero; handing the device's gate pattern to the checker separates that effect
        # from the arithmetic of the kernels under test.
        self.relu_gates = None

    # tensor.dart:867-947
    def matMul(self, a, b):
        out = T(self.ops.matmul_fwd(a.value, b.value))
        return _node(out, [a, b], lambda: self.ops.matmul_bwd(a.value, b.value, out.grad, a.grad, b.grad))

    # tensor.dart:679-709
    def addMatrixAndVector(self, m, v):
        out = T(m.value + v.value[None, :])

        def bw():
            m.grad += out.grad
            for i in range(out.grad.shape[0]):  # row order, as the reference's i-outer loop
                v.grad += out.grad[i]
        return _node(out, [m, v], bw)

    # tensor.dart:651-677
    def addMatrix(self, a, b):
        out = T(a.value + b.value)

        def bw():
            a.grad += out.grad
            b.grad += out.grad
        return _node(out, [a, b], bw)

    def _unary(self, name, x, saved_is_output):
        out = T(self.ops.unary_fwd(name, x.value))
        saved = out.value if saved_is_output else x.value
        return _node(out, [x], lambda: self.ops.unary_bwd(name, saved, out.grad, x.grad))

    def reluMatrix(self, x):      # tensor.dart:1013-1038
        if self.relu_gates is not None:
            gate = np.asarray(next(self.relu_gates), dtype=np.float64)
            out = T(x.value * gate)

            def bw():
                x.grad += out.grad * gate
            return _node(out, [x], bw)
        return self._unary("relu", x, False)

    def sigmoidMatrix(self, x):   # tensor.dart:1123-1151
        return self._unary("sigmoid", x, True)

    def tanhMatrix(self, x):      # tensor.dart:1178-1209
        return self._unary("tanh", x, True)

    def geluMatrix(self, x):      # EXTENSION
        return self._unary("gelu", x, False)

    # tensor.dart:1075-1101
    def scaleMatrix(self, x, s):
        out = T(x.value * s)

        def bw():
            x.grad += out.grad * s
        return _node(out, [x], bw)

    # tensor.dart:1211-1236
    def transpose(self, x):
        out = T(x.value.T.copy())

        def bw():
            x.grad += out.grad.T
        return _node(out, [x], bw)

    # tensor.dart:739-763
    def concatenateMatricesByColumn(self, parts):
        out = T(np.concatenate([p.value for p in parts], axis=1))

        def bw():
            c = 0
            for p in parts:
                w = p.value.shape[1]
                p.grad += out.grad[:, c:c + w]
                c += w
        return _node(out, parts, bw)

    # lib/activationFunctions/softmax.dart:68-115 (+ causal EXTENSION)
    def softmaxMatrix(self, x, causal=False):
        out = T(self.ops.softmax_fwd(x.value, x.value.shape[0] if causal else 0))
        return _node(out, [x], lambda: self.ops.softmax_bwd(out.value, out.grad, x.grad))

    # lib/transformer/layerNormalization.dart:137-202
    def layerNorm(self, x, gamma, beta, eps=1e-5):
        y, xhat, var = self.ops.layernorm_fwd(x.value, gamma.value, beta.value, eps)
        out = T(y)
        return _node(out, [x, gamma, beta], lambda: self.ops.layernorm_bwd(
            out.grad, gamma.value, xhat, var, x.grad, gamma.grad, beta.grad, eps))

    # tensor.dart:982-1011
    def mseMatrix(self, p, t):
        out = T(np.array(self.ops.mse_fwd(p.value, t.value)))
        return _node(out, [p], lambda: self.ops.mse_bwd(p.value, t.value, p.grad, float(out.grad)))

    # EXTENSION
    def softmaxCrossEntropy(self, z, labels, inv_count):
        out = T(np.array(self.ops.softmax_xent(z.value, labels, None, inv_count)))

        def bw():
            dz = np.zeros_like(z.value)
            self.ops.softmax_xent(z.value, labels, dz, inv_count)
            z.grad += float(out.grad) * dz
        return _node(out, [z], bw)

    # lib/transformer/embeddingLayer.dart:47-67
    def embedding(self, table, ids):
        out = T(self.ops.embedding_fwd(table.value, ids))
        return _node(out, [table], lambda: self.ops.embedding_bwd(out.grad, ids, table.grad))

    # tensor.dart:765-833; padding 'valid' or 'same'
    def conv2d(self, x, k, padding="valid"):
        pad = (k.value.shape[0] - 1) // 2 if padding == "same" else 0
        out = T(self.ops.conv2d_fwd(x.value, k.value, pad))
        return _node(out, [x, k], lambda: self.ops.conv2d_bwd(x.value, k.value, out.grad, x.grad, k.grad, pad))

    # tensor.dart:711-737: m + s for a scalar tensor s; s.grad += sum of out.grad
    def addScalarToMatrix(self, m, s):
        out = T(m.value + float(np.asarray(s.value).reshape(-1)[0]))

        def bw():
            m.grad += out.grad
            s.grad += out.grad.sum()
        return _node(out, [m, s], bw)

    # tensor.dart:949-980
    def matVecMul(self, M, v):
        out = T(self.ops.matvec_fwd(M.value, v.value))
        return _node(out, [M, v], lambda: self.ops.matvec_bwd(M.value, v.value, out.grad, M.grad, v.grad))

    # tensor.dart:478-497 (vector), 835-865 (matrix)
    def elementWiseMultiply(self, a, b):
        out = T(a.value * b.value)

        def bw():
            a.grad += out.grad * b.value
            b.grad += out.grad * a.value
        return _node(out, [a, b], bw)

    # tensor.dart:561-579 (sum), 1153-1176 (sumMatrix): row-major running total
    def sum(self, x):
        total = 0.0
        for v in x.value.ravel():
            total += v
        out = T(np.array(total))

        def bw():
            x.grad += float(out.grad)
        return _node(out, [x], bw)

    # lib/activationFunctions/{leakyRelu,elu,silu,mish}.dart (kinds 5..8 of orc_act2_*)
    def act2(self, kind, x, alpha=0.0):
        out = T(self.ops.act2_fwd(kind, alpha, x.value))
        return _node(out, [x], lambda: self.ops.act2_bwd(kind, alpha, x.value, out.grad, x.grad))

    # tensor.dart:437-455
    def concatenate(self, a, b):
        out = T(np.concatenate([a.value, b.value]))

        def bw():
            a.grad += out.grad[:a.value.size]
            b.grad += out.grad[a.value.size:]
        return _node(out, [a, b], bw)

    # ---------------------------------------------------------------- layers

    def dense_matrix(self, x, W, b, act=None):
        """DenseLayerMatrix.forward lib/layertypes/denseLayer.dart:116-125: act(X.W + b),
        W stored [in x out] (:96-104)."""
        z = self.addMatrixAndVector(self.matMul(x, W), b)
        if act is None:
            return z
        return {"relu": self.reluMatrix, "sigmoid": self.sigmoidMatrix, "tanh": self.tanhMatrix,
                "gelu": self.geluMatrix}[act](z)

    def single_head(self, x, Wq, Wk, Wv, causal):
        """SingleHeadAttention.forward lib/layertypes/singleHeadAttentionLayer.dart:70-89."""
        Q, K, V = self.matMul(x, Wq), self.matMul(x, Wk), self.matMul(x, Wv)
        scores = self.matMul(Q, self.transpose(K))
        scaled = self.scaleMatrix(scores, 1 / math.sqrt(Wq.value.shape[1]))
        P = self.softmaxMatrix(scaled, causal)
        return self.matMul(P, V)

    def multi_head(self, x, heads, Wo, causal):
        """MultiHeadAttention.forward lib/transformer/multiHeadAttentionLayer.dart:72-84:
        heads serially, column concat, then .Wo (no biases anywhere)."""
        outs = [self.single_head(x, *h, causal) for h in heads]
        return self.matMul(self.concatenateMatricesByColumn(outs), Wo)

    def encoder_block(self, x, p, causal):
        """TransformerEncoderBlock.forward lib/transformer/transformerEncodingLayer.dart:58-70
        (post-LN; FFN = Dense(dff, ReLU) -> Dense(dModel), :48-51)."""
        attn = self.multi_head(x, p["heads"], p["Wo"], causal)
        h = self.layerNorm(self.addMatrix(x, attn), p["g1"], p["be1"])
        f = self.dense_matrix(self.dense_matrix(h, p["W1"], p["b1"], "relu"), p["W2"], p["b2"])
        return self.layerNorm(self.addMatrix(h, f), p["g2"], p["be2"])


def block_params_to_T(p):
    """Wrap a dict of numpy arrays (heads: list of (Wq,Wk,Wv)) into tape tensors."""
    out = {k: T(v) for k, v in p.items() if k != "heads"}
    out["heads"] = [tuple(T(w) for w in h) for h in p["heads"]]
    return out


def block_param_list(pt):
    lst = []
    for h in pt["heads"]:
        lst += list(h)
    return lst + [pt[k] for k in ("Wo", "g1", "be1", "W1", "b1", "W2", "b2", "g2", "be2")]


# ------------------------------------------------------------------ config drivers


def mlp_step(X, labels, params, lr=0.01, omp=False):
    """Config 1: DenseLayerMatrix(128,ReLU) -> (64,ReLU) -> (10) -> softmax-CE (mean over
    the batch) -> backward -> SGD (lib/nets/snet.dart:74-85 order: forward, loss,
    backward, step).  params = [W1,b1,W2,b2,W3,b3] float64."""
    E = Engine(omp)
    P = [T(p) for p in params]
    x = T(X)
    h1 = E.dense_matrix(x, P[0], P[1], "relu")
    h2 = E.dense_matrix(h1, P[2], P[3], "relu")
    logits = E.dense_matrix(h2, P[4], P[5])
    loss = E.softmaxCrossEntropy(logits, labels, 1.0 / X.shape[0])
    loss.backward()
    grads = [p.grad.copy() for p in P]
    new = []
    for p in P:
        w = p.value.copy()
        E.ops.sgd_step(w, p.grad, lr)
        new.append(w)
    return {"logits": logits.value, "loss": float(loss.value), "grads": grads, "params": new}


def gemm_gelu_fwd_bwd(A, B, bias, dC, omp=False):
    """Config 2: Z=A.B+bias, C=GELU(Z); dZ=dC*GELU'(Z); dA=dZ.B^T; dB=A^T.dZ; dbias."""
    E = Engine(omp)
    a, b, bi = T(A), T(B), T(bias)
    z = E.addMatrixAndVector(E.matMul(a, b), bi)
    c = E.geluMatrix(z)
    c.grad = np.ascontiguousarray(dC, dtype=np.float64)
    for node in (c, z):
        node.backward_fn()
    mm = z.inputs[0]
    mm.backward_fn()
    return {"Z": z.value, "C": c.value, "dZ": z.grad, "dA": a.grad, "dB": b.grad, "dbias": bi.grad}


def encoder_block_fwd_bwd(xs, params, targets, causal=True, omp=False, relu_gates=None):
    """Config 3: one post-LN block over a batch of sequences.  Each sequence is one
    reference forward/backward (mseMatrix against its target); gradients accumulate
    across sequences and the reported loss is the sum.  `relu_gates` (one boolean mask
    [seq x dff] per sequence) replaces the FFN's own gate pattern, see Engine.relu_gates."""
    E = Engine(omp)
    if relu_gates is not None:
        E.relu_gates = iter(relu_gates)
    pt = block_params_to_T(params)
    ys, loss, dxs = [], 0.0, []
    for x_np, t_np in zip(xs, targets):
        x = T(x_np)
        y = E.encoder_block(x, pt, causal)
        l = E.mseMatrix(y, T(t_np))
        l.backward()
        ys.append(y.value)
        dxs.append(x.grad)
        loss += float(l.value)
    return {"y": np.stack(ys), "loss": loss, "dx": np.stack(dxs),
            "grads": [p.grad for p in block_param_list(pt)]}


def lm_forward_backward(ids, labels, params, n_global_tokens, causal=True, omp=False):
    """Config 5 (one data-parallel shard): Embedding -> +PositionalEncoding -> blocks ->
    DenseLayerMatrix(vocab) -> softmax-CE normalised by the GLOBAL token count.
    ids/labels [B,S] ints.  Returns loss contribution and gradients in parameter order
    [emb, (block params)*, Whead, bhead]."""
    E = Engine(omp)
    emb = T(params["emb"])
    blocks = [block_params_to_T(b) for b in params["blocks"]]
    Wh, bh = T(params["Whead"]), T(params["bhead"])
    S = ids.shape[1]
    pe = T(E.ops.positional_table(S, emb.value.shape[1]))
    loss = 0.0
    logits_all = []
    for b in range(ids.shape[0]):
        h = E.addMatrix(E.embedding(emb, ids[b].astype(np.float64)), pe)
        for bp in blocks:
            h = E.encoder_block(h, bp, causal)
        logits = E.dense_matrix(h, Wh, bh)
        l = E.softmaxCrossEntropy(logits, labels[b], 1.0 / n_global_tokens)
        l.backward()
        loss += float(l.value)
        logits_all.append(logits.value)
    plist = [emb]
    for bp in blocks:
        plist += block_param_list(bp)
    plist += [Wh, bh]
    return {"loss": loss, "logits": np.stack(logits_all), "grads": [p.grad for p in plist],
            "params": [p.value for p in plist]}


def tiered_lstm_fwd_bwd(x, Ws, bs, cycles, target, dual=False, omp=False):
    """MultiTierLSTMLayer.forward (lib/layertypes/multilstm.dart:111-167) or, with `dual`, DualLSTMLayer.forward
    (lib/layertypes/duallstm.dart:98-175) for ONE sequence x [T x I], composed from the tape's vector operations the way
    the reference composes them (concatenate :437-455, matVecMul :949-980, addVector :395-414, sigmoid :541-559,
    vectorTanh :581-605, elementWiseMultiply :478-497 of lib/autogradEngine/tensor.dart), then mse against `target`
    (tensor.dart:499-519) and the tape's backward sweep.  Ws[i] is [4H x combined_i], the four gate matrices of tier i
    stacked f, i, c~, o; bs[i] is [4H].  Returns the last hidden state of tier 0, the loss, dWs, dbs and dx."""
    e = Engine(omp)
    n = len(cycles) + 1
    H = Ws[0].shape[0] // 4
    cum, prod = [], 1
    for c in cycles:
        prod *= c
        cum.append(prod)
    Wt = [[T(W[g * H:(g + 1) * H]) for g in range(4)] for W in Ws]
    bt = [[T(b[g * H:(g + 1) * H]) for g in range(4)] for b in bs]
    xs = [T(row) for row in np.asarray(x, dtype=np.float64)]
    h = [T(np.zeros(H)) for _ in range(n)]
    c_ = [T(np.zeros(H)) for _ in range(n)]

    def step(combined, c_prev, tier):     # multilstm.dart:160-178
        W, b = Wt[tier], bt[tier]
        f = e._unary("sigmoid", e.addMatrix(e.matVecMul(W[0], combined), b[0]), True)
        i = e._unary("sigmoid", e.addMatrix(e.matVecMul(W[1], combined), b[1]), True)
        g = e._unary("tanh", e.addMatrix(e.matVecMul(W[2], combined), b[2]), True)
        c_next = e.addMatrix(e.elementWiseMultiply(f, c_prev), e.elementWiseMultiply(i, g))
        o = e._unary("sigmoid", e.addMatrix(e.matVecMul(W[3], combined), b[3]), True)
        return e.elementWiseMultiply(o, e._unary("tanh", c_next, True)), c_next

    for t, x_t in enumerate(xs):
        combined = h[0]
        for j in range(1, n):             # [h_0, c_1, ..., c_{n-1}, x_t]  (multilstm.dart:137-150, duallstm.dart:116-117)
            combined = e.concatenate(combined, c_[j])
        combined = e.concatenate(combined, x_t)
        h[0], c_[0] = step(combined, c_[0], 0)
        for i in range(1, n):
            fires = (t + 1) % cum[i - 1] == 0 and (t > 0 or not dual)     # multilstm.dart:155, duallstm.dart:145
            if fires:
                h[i], c_[i] = step(e.concatenate(h[i], h[i - 1]), c_[i], i)
    out = h[0]
    loss = e.mseMatrix(out, T(target))
    loss.backward()
    dWs = [np.concatenate([w.grad for w in W], axis=0) for W in Wt]
    dbs = [np.concatenate([v.grad for v in b]) for b in bt]
    return out.value.copy(), float(loss.value), dWs, dbs, np.stack([v.grad for v in xs])


def conv_lstm_fwd_bwd(x, Kx, Kh, bias, target, omp=False):
    """ConvLSTMLayer.forward (lib/layertypes/convlstmLayer.dart:107-159) for ONE sequence of frames x [T x H x W], composed
    from the tape's operations the way the reference composes them (conv2d with 'same' padding tensor.dart:765-833,
    addMatrix :651-677, sigmoidMatrix :1123-1151, tanhMatrix :1178-1209, elementWiseMultiplyMatrix :835-865), then
    mseMatrix against `target` [H x W] (:982-1011) and the tape's backward sweep.  Kx, Kh are [4 x k x k] (the input and
    hidden kernels of the gates f, i, c~, o), bias is [4 x H x W] (one bias MATRIX per gate, :83-96).  Returns the last
    hidden map, the loss, dKx, dKh, dbias and dx."""
    e = Engine(omp)
    kx = [T(k) for k in np.asarray(Kx, dtype=np.float64)]
    kh = [T(k) for k in np.asarray(Kh, dtype=np.float64)]
    bs = [T(b) for b in np.asarray(bias, dtype=np.float64)]
    xs = [T(f) for f in np.asarray(x, dtype=np.float64)]
    H, W = xs[0].value.shape
    h, c = T(np.zeros((H, W))), T(np.zeros((H, W)))

    def gate(g, x_t, act):
        z = e.addMatrix(e.addMatrix(e.conv2d(x_t, kx[g], "same"), e.conv2d(h, kh[g], "same")), bs[g])
        return e._unary(act, z, True)

    for x_t in xs:
        f = gate(0, x_t, "sigmoid")
        i = gate(1, x_t, "sigmoid")
        g = gate(2, x_t, "tanh")
        c = e.addMatrix(e.elementWiseMultiply(f, c), e.elementWiseMultiply(i, g))
        o = gate(3, x_t, "sigmoid")
        h = e.elementWiseMultiply(o, e._unary("tanh", c, True))
    loss = e.mseMatrix(h, T(target))
    loss.backward()
    return (h.value.copy(), float(loss.value), np.stack([k.grad for k in kx]), np.stack([k.grad for k in kh]),
            np.stack([b.grad for b in bs]), np.stack([v.grad for v in xs]))


def chained_scale_fwd_bwd(x, Ws, bs, aWs, abs_, grains, final_len, target, lookback=10, omp=False):
    """GeneralizedChainedScaleLayer.forward (lib/layertypes/trendmodelLayer.dart:134-204) for ONE sequence x [T x I], composed
    from the tape's vector operations as the reference composes them: every complete chunk of grain_i consecutive
    vectors of level i is flattened (concatenate, tensor.dart:437-455) and summarised by vectorTanh(aggW_i . chunk +
    aggB_i) (:146-158); then one LSTM loop per level from the highest down (:163-178, :181-204), each over at most
    `lookback` (level 0: `final_len`) of its most recent inputs, its hidden state initialised with the level above's
    result, its cell state with zeros; mse against `target`; the tape's backward sweep.  Ws[i] = [4H x (H + I)] (gates f, i,
    c~, o stacked, columns [h | x]), bs[i] = [4H], aWs[i] = [I x grain_i * I], abs_[i] = [I].
    Returns h, loss, dWs, dbs, daWs, dabs, dx."""
    e = Engine(omp)
    n = len(grains) + 1
    H = Ws[0].shape[0] // 4
    Wt = [[T(W[g * H:(g + 1) * H]) for g in range(4)] for W in Ws]
    bt = [[T(b[g * H:(g + 1) * H]) for g in range(4)] for b in bs]
    aWt, abt = [T(w) for w in aWs], [T(b) for b in abs_]
    xs = [T(row) for row in np.asarray(x, dtype=np.float64)]
    tier_inputs = [xs[len(xs) - final_len:]] + [[] for _ in range(n - 1)]
    current = xs
    for i, grain in enumerate(grains):
        nxt = []
        for j in range(0, len(current) - grain + 1, grain):
            flat = current[j]
            for v in current[j + 1:j + grain]:
                flat = e.concatenate(flat, v)
            nxt.append(e._unary("tanh", e.addMatrix(e.matVecMul(aWt[i], flat), abt[i]), True))
        tier_inputs[i + 1] = nxt
        current = nxt
    context = T(np.zeros(H))
    for i in range(n - 1, -1, -1):
        seq = tier_inputs[i]
        look = final_len if i == 0 else lookback
        seq = seq[max(0, len(seq) - look):]
        h, c = context, T(np.zeros(H))
        W, b = Wt[i], bt[i]
        for x_t in seq:
            comb = e.concatenate(h, x_t)
            f = e._unary("sigmoid", e.addMatrix(e.matVecMul(W[0], comb), b[0]), True)
            ig = e._unary("sigmoid", e.addMatrix(e.matVecMul(W[1], comb), b[1]), True)
            g = e._unary("tanh", e.addMatrix(e.matVecMul(W[2], comb), b[2]), True)
            c = e.addMatrix(e.elementWiseMultiply(f, c), e.elementWiseMultiply(ig, g))
            o = e._unary("sigmoid", e.addMatrix(e.matVecMul(W[3], comb), b[3]), True)
            h = e.elementWiseMultiply(o, e._unary("tanh", c, True))
        context = h
    loss = e.mseMatrix(context, T(target))
    loss.backward()
    return (context.value.copy(), float(loss.value), [np.concatenate([w.grad for w in W], axis=0) for W in Wt],
            [np.concatenate([v.grad for v in b]) for b in bt], [w.grad for w in aWt], [b.grad for b in abt], np.stack([v.grad for v in xs]))
