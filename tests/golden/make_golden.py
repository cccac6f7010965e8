"""Regenerates tests/golden/*.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference's Dart engine cannot be executed in this environment, so these vectors are outputs of
the float64 restatement (oracle/), not of the reference itself: they freeze the oracle's behaviour
(a change in oracle.c that alters any number shows up as a test failure) and give the GPU tests
fixed targets that do not depend on the oracle being rebuilt.  Inputs come from the seeded generator
and are stored as float32, outputs as float64.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from flutter_ml_b200 import synth  # noqa: E402
from oracle import oracle  # noqa: E402

w64 = lambda x: np.ascontiguousarray(x, dtype=np.float64)  # noqa: E731


def gemm_gelu():
    M, K, N = 48, 40, 32
    A, B = synth.normal(1, 0, (M, K), 1 / np.sqrt(K)), synth.normal(1, 1, (K, N), 1 / np.sqrt(K))
    bias, dC = synth.normal(1, 2, (N,), 1 / np.sqrt(K)), synth.normal(1, 3, (M, N), 1 / np.sqrt(K))
    o = oracle.gemm_gelu_fwd_bwd(w64(A), w64(B), w64(bias), w64(dC))
    np.savez_compressed(os.path.join(HERE, "gemm_gelu_48x32x40.npz"), A=A, B=B, bias=bias, dC=dC, **o)


def mlp():
    sizes = (32, 16, 12, 5)
    params = []
    for i, (a, b) in enumerate(zip(sizes[:-1], sizes[1:])):
        params += [synth.xavier_uniform(0, 10 + i, a, b), np.zeros(b, np.float32)]
    X, labels = synth.uniform(0, 0, (8, sizes[0])), synth.integers(0, 1, (8,), sizes[-1])
    o = oracle.mlp_step(w64(X), labels, [w64(p) for p in params], lr=0.01)
    d = {"X": X, "labels": labels, "logits": o["logits"], "loss": np.array(o["loss"])}
    for i, (p, g, n) in enumerate(zip(params, o["grads"], o["params"])):
        d[f"p{i}"], d[f"g{i}"], d[f"n{i}"] = p, g, n
    np.savez_compressed(os.path.join(HERE, "mlp_32_16_12_5.npz"), **d)


def lstm():
    T, B, I, H = 5, 3, 8, 12
    a = 1 / np.sqrt(H)
    W, b = synth.uniform(3, 0, (4, H, H + I), -a, a), synth.uniform(3, 1, (4, H), -0.1, 0.1)
    x, target = synth.normal(3, 2, (B, T, I)), synth.normal(3, 3, (B, H))
    h, loss, dW, db = oracle.Ops().lstm_fwd_bwd(w64(W), w64(b), w64(x), w64(target))
    np.savez_compressed(os.path.join(HERE, "lstm_T5_B3_I8_H12.npz"), W=W, b=b, x=x, target=target, h_last=h,
                        loss=np.array(loss), dW=dW, db=db)


def rows():
    x = synth.normal(5, 0, (6, 16), 2.0)
    g, be, dy = 1 + synth.normal(5, 1, (16,), 0.1), synth.normal(5, 2, (16,), 0.1), synth.normal(5, 3, (6, 16))
    ops = oracle.Ops()
    sm = ops.softmax_fwd(w64(x), 6)
    dsm = np.zeros_like(sm)
    ops.softmax_bwd(sm, w64(dy), dsm)
    y, xhat, var = ops.layernorm_fwd(w64(x), w64(g), w64(be))
    dx, dg, db = np.zeros_like(y), np.zeros(16), np.zeros(16)
    ops.layernorm_bwd(w64(dy), w64(g), xhat, var, dx, dg, db)
    np.savez_compressed(os.path.join(HERE, "rows_6x16.npz"), x=x, gamma=g, beta=be, dy=dy, softmax_causal=sm,
                        softmax_bwd=dsm, ln_y=y, ln_dx=dx, ln_dgamma=dg, ln_dbeta=db)


def widened():
    """The later additions in one file: the six optimizer rules over three steps, the four parameterised activations,
    conv2d ('same', 3 x 3) with its gradients, and one causal attention head (output and dQ, dK, dV)."""
    ops = oracle.Ops()
    d = {}
    n = 37
    w0 = synth.normal(7, 0, (n,))
    grads = [synth.normal(7, 1 + t, (n,)) for t in range(3)]
    d["opt_w0"], d["opt_grads"] = w0, np.stack(grads)
    for kind, h, nstate in ((1, (0.9,), 1), (2, (0.9,), 1), (3, (0.9, 1e-8), 1), (4, (0.0, 1e-8), 1),
                            (6, (0.9, 0.999, 1e-8, 0.01), 2), (7, (0.9, 0.999, 1e-8), 3)):
        w = w64(w0)
        st = [np.zeros(n) for _ in range(nstate)] + [None] * (3 - nstate)
        for t, g in enumerate(grads, 1):
            ops.optimizer_step(kind, w, w64(g), st[0], st[1], st[2], 0.01, h, t)
        d[f"opt_w_kind{kind}"] = w
    x = synth.normal(7, 10, (64,), 3.0)
    dy = synth.normal(7, 11, (64,))
    d["act_x"], d["act_dy"] = x, dy
    for kind, alpha in ((5, 0.01), (6, 1.0), (7, 0.0), (8, 0.0)):
        d[f"act_y_kind{kind}"] = ops.act2_fwd(kind, alpha, w64(x))
        dx = np.zeros(64)
        ops.act2_bwd(kind, alpha, w64(x), w64(dy), dx)
        d[f"act_dx_kind{kind}"] = dx
    img, ker, dout = synth.normal(7, 20, (9, 11)), synth.normal(7, 21, (3, 3)), synth.normal(7, 22, (9, 11))
    d["conv_x"], d["conv_k"], d["conv_dout"] = img, ker, dout
    d["conv_out"] = ops.conv2d_fwd(w64(img), w64(ker), 1)
    dimg, dker = np.zeros((9, 11)), np.zeros((3, 3))
    ops.conv2d_bwd(w64(img), w64(ker), w64(dout), dimg, dker, 1)
    d["conv_dx"], d["conv_dk"] = dimg, dker
    S, dk = 128, 64
    Q, K, V, G = (synth.normal(7, 30 + i, (S, dk)) for i in range(4))
    E = oracle.Engine()
    tq, tk, tv = oracle.T(w64(Q)), oracle.T(w64(K)), oracle.T(w64(V))
    O = E.matMul(E.softmaxMatrix(E.scaleMatrix(E.matMul(tq, E.transpose(tk)), 0.125), True), tv)
    E.sum(E.elementWiseMultiply(O, oracle.T(w64(G)))).backward()
    d.update(att_q=Q, att_k=K, att_v=V, att_g=G, att_out=O.value, att_dq=tq.grad, att_dk=tk.grad, att_dv=tv.grad)
    np.savez_compressed(os.path.join(HERE, "widened_ops.npz"), **d)


if __name__ == "__main__":
    oracle.build()
    gemm_gelu(); mlp(); lstm(); rows(); widened()
    print(sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
