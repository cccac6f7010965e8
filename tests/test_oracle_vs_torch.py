"""Independent check of the oracle: the same math written with torch float64 autograd."""
import math

import numpy as np
import pytest
import torch

torch.set_default_dtype(torch.float64)
TOL = 1e-11


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def tt(x, grad=True):
    return torch.tensor(np.asarray(x, dtype=np.float64), requires_grad=grad)


def t_ln(x, g, b, eps=1e-5):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return g * (x - mu) / torch.sqrt(var + eps) + b


def t_block(x, p, causal):
    outs = []
    S = x.shape[0]
    for Wq, Wk, Wv in p["heads"]:
        s = (x @ Wq) @ (x @ Wk).T * (1 / math.sqrt(Wq.shape[1]))
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -float("inf"))
        outs.append(torch.softmax(s, -1) @ (x @ Wv))
    attn = torch.cat(outs, 1) @ p["Wo"]
    h = t_ln(x + attn, p["g1"], p["be1"])
    f = torch.relu(h @ p["W1"] + p["b1"]) @ p["W2"] + p["b2"]
    return t_ln(h + f, p["g2"], p["be2"])


def make_block(rng, d, heads, dff):
    dk = d // heads
    return {"heads": [tuple(rng.normal(0, 0.2, (d, dk)) for _ in range(3)) for _ in range(heads)],
            "Wo": rng.normal(0, 0.2, (d, d)), "g1": 1 + 0.1 * rng.normal(size=d), "be1": 0.1 * rng.normal(size=d),
            "W1": rng.normal(0, 0.2, (d, dff)), "b1": 0.1 * rng.normal(size=dff),
            "W2": rng.normal(0, 0.2, (dff, d)), "b2": 0.1 * rng.normal(size=d),
            "g2": 1 + 0.1 * rng.normal(size=d), "be2": 0.1 * rng.normal(size=d)}


def block_to_torch(p):
    q = {k: tt(v) for k, v in p.items() if k != "heads"}
    q["heads"] = [tuple(tt(w) for w in h) for h in p["heads"]]
    return q


def torch_block_list(q):
    lst = []
    for h in q["heads"]:
        lst += list(h)
    return lst + [q[k] for k in ("Wo", "g1", "be1", "W1", "b1", "W2", "b2", "g2", "be2")]


def test_mlp_step(orc):
    rng = np.random.default_rng(0)
    X = rng.uniform(size=(16, 20))
    labels = rng.integers(0, 5, 16)
    shapes = [(20, 12), (12,), (12, 8), (8,), (8, 5), (5,)]
    params = [rng.normal(0, 0.3, s) for s in shapes]
    o = orc.mlp_step(X, labels, params, lr=0.01)
    P = [tt(p) for p in params]
    h = torch.relu(tt(X, False) @ P[0] + P[1])
    h = torch.relu(h @ P[2] + P[3])
    logits = h @ P[4] + P[5]
    loss = torch.nn.functional.cross_entropy(logits, torch.tensor(labels))
    loss.backward()
    assert abs(o["loss"] - loss.item()) < 1e-12
    assert rel(o["logits"], logits.detach().numpy()) < TOL
    for g, p, w in zip(o["grads"], P, o["params"]):
        assert rel(g, p.grad.numpy()) < TOL
        assert rel(w, (p - 0.01 * p.grad).detach().numpy()) < TOL


def test_gemm_gelu(orc):
    rng = np.random.default_rng(1)
    M, K, N = 9, 13, 7
    A, B, bias, dC = rng.normal(size=(M, K)), rng.normal(size=(K, N)), rng.normal(size=N), rng.normal(size=(M, N))
    o = orc.gemm_gelu_fwd_bwd(A, B, bias, dC)
    a, b, bi = tt(A), tt(B), tt(bias)
    z = a @ b + bi
    z.retain_grad()
    c = torch.nn.functional.gelu(z)
    c.backward(tt(dC, False))
    assert rel(o["C"], c.detach().numpy()) < TOL
    for k, t in (("dZ", z.grad), ("dA", a.grad), ("dB", b.grad), ("dbias", bi.grad)):
        assert rel(o[k], t.numpy()) < TOL, k


@pytest.mark.parametrize("causal", [False, True])
def test_encoder_block(orc, causal):
    rng = np.random.default_rng(2)
    d, heads, dff, S, B = 16, 4, 24, 10, 3
    p = make_block(rng, d, heads, dff)
    xs, ts = rng.normal(size=(B, S, d)), rng.normal(size=(B, S, d))
    o = orc.encoder_block_fwd_bwd(xs, p, ts, causal)
    q = block_to_torch(p)
    X = tt(xs)
    total = 0
    ys = []
    for b in range(B):
        y = t_block(X[b], q, causal)
        ys.append(y)
        total = total + ((y - tt(ts[b], False)) ** 2).mean()
    total.backward()
    assert abs(o["loss"] - total.item()) < 1e-11
    assert rel(o["y"], torch.stack(ys).detach().numpy()) < TOL
    assert rel(o["dx"], X.grad.numpy()) < 1e-10
    for g, t in zip(o["grads"], torch_block_list(q)):
        assert rel(g, t.grad.numpy()) < 1e-10


def test_lstm(orc):
    rng = np.random.default_rng(3)
    B, T, I, H = 3, 6, 5, 7
    W = rng.uniform(-0.4, 0.4, (4, H, H + I))
    b = rng.uniform(-0.1, 0.1, (4, H))
    x, target = rng.normal(size=(B, T, I)), rng.normal(size=(B, H))
    h_last, loss, dW, db = orc.Ops().lstm_fwd_bwd(W, b, x, target)
    Wt, bt = tt(W), tt(b)
    total = 0
    hs = []
    for s in range(B):
        h, c = torch.zeros(H), torch.zeros(H)
        for t in range(T):
            z = torch.cat([h, tt(x[s, t], False)])
            f = torch.sigmoid(Wt[0] @ z + bt[0])
            i = torch.sigmoid(Wt[1] @ z + bt[1])
            g = torch.tanh(Wt[2] @ z + bt[2])
            c = f * c + i * g
            o = torch.sigmoid(Wt[3] @ z + bt[3])
            h = o * torch.tanh(c)
        hs.append(h)
        total = total + ((h - tt(target[s], False)) ** 2).mean()
    total.backward()
    assert abs(loss - total.item()) < 1e-12
    assert rel(h_last, torch.stack(hs).detach().numpy()) < TOL
    assert rel(dW, Wt.grad.numpy()) < 1e-10 and rel(db, bt.grad.numpy()) < 1e-10


def test_lm_step_and_adam(orc):
    rng = np.random.default_rng(4)
    V, d, heads, dff, S, B, L = 30, 16, 4, 24, 8, 3, 2
    params = {"emb": rng.normal(0, 0.3, (V, d)), "blocks": [make_block(rng, d, heads, dff) for _ in range(L)],
              "Whead": rng.normal(0, 0.3, (d, V)), "bhead": 0.1 * rng.normal(size=V)}
    ids, labels = rng.integers(0, V, (B, S)), rng.integers(0, V, (B, S))
    o = orc.lm_forward_backward(ids, labels, params, B * S)
    emb, Wh, bh = tt(params["emb"]), tt(params["Whead"]), tt(params["bhead"])
    blocks = [block_to_torch(b) for b in params["blocks"]]
    pos = torch.arange(S, dtype=torch.float64)[:, None]
    i = torch.arange(d, dtype=torch.float64)[None, :]
    ang = pos / torch.pow(torch.tensor(10000.0), 2 * i / d)
    pe = torch.where((torch.arange(d) % 2 == 0)[None, :], torch.sin(ang), torch.cos(ang))
    total = 0
    for b in range(B):
        h = emb[torch.tensor(ids[b])] + pe
        for q in blocks:
            h = t_block(h, q, True)
        logits = h @ Wh + bh
        total = total + torch.nn.functional.cross_entropy(logits, torch.tensor(labels[b]), reduction="sum") / (B * S)
    total.backward()
    plist = [emb] + sum((torch_block_list(q) for q in blocks), []) + [Wh, bh]
    assert abs(o["loss"] - total.item()) < 1e-11
    for g, t in zip(o["grads"], plist):
        assert rel(g, t.grad.numpy()) < 1e-10
    # Adam (lib/optimizers/adam.dart:44-77) against torch.optim.Adam for two steps
    ops = orc.Ops()
    w = params["Whead"].copy()
    g = o["grads"][-2]
    m, v = np.zeros_like(w), np.zeros_like(w)
    wt = tt(params["Whead"])
    opt = torch.optim.Adam([wt], lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
    for t in (1, 2):
        ops.adam_step(w, g, m, v, 1e-3, t)
        wt.grad = tt(g, False)
        opt.step()
    assert rel(w, wt.detach().numpy()) < 1e-12


def test_finite_difference_layernorm_softmax(orc):
    rng = np.random.default_rng(5)
    ops = orc.Ops()
    x, g, b = rng.normal(size=(4, 9)), rng.normal(size=9), rng.normal(size=9)
    w = rng.normal(size=(4, 9))

    def f(xx):
        y, _, _ = ops.layernorm_fwd(xx, g, b)
        return float((ops.softmax_fwd(y, 4) * w).sum())
    y, xhat, var = ops.layernorm_fwd(x, g, b)
    s = ops.softmax_fwd(y, 4)
    dy = np.zeros_like(x)
    ops.softmax_bwd(s, w, dy)
    dx = np.zeros_like(x)
    ops.layernorm_bwd(dy, g, xhat, var, dx, np.zeros(9), np.zeros(9))
    num = np.zeros_like(x)
    for idx in np.ndindex(*x.shape):
        xp, xm = x.copy(), x.copy()
        xp[idx] += 1e-6
        xm[idx] -= 1e-6
        num[idx] = (f(xp) - f(xm)) / 2e-6
    assert rel(dx, num) < 1e-6


@pytest.mark.parametrize("kind,alpha,fn", [
    (5, 0.01, lambda x: torch.nn.functional.leaky_relu(x, 0.01)),
    (5, 0.3, lambda x: torch.nn.functional.leaky_relu(x, 0.3)),
    (6, 1.0, lambda x: torch.nn.functional.elu(x, 1.0)),
    (6, 0.5, lambda x: torch.nn.functional.elu(x, 0.5)),
    (7, 0.0, torch.nn.functional.silu),
    (8, 0.0, torch.nn.functional.mish),
])
def test_parameterised_activations(orc, kind, alpha, fn):
    rng = np.random.default_rng(kind)
    x = np.concatenate([rng.standard_normal(500) * 3, [0.0, -30.0, 30.0, 400.0, -400.0]])
    dy = rng.standard_normal(x.size)
    ops = orc.Ops()
    y = ops.act2_fwd(kind, alpha, x)
    dx = np.zeros_like(x)
    ops.act2_bwd(kind, alpha, x, dy, dx)
    xt = tt(x)
    yt = fn(xt)
    yt.backward(torch.tensor(dy))
    assert rel(y, yt.detach().numpy()) <= 1e-12
    assert rel(dx, xt.grad.numpy()) <= 1e-12
    # backward accumulates (+=), as every tape closure of the reference does
    ops.act2_bwd(kind, alpha, x, dy, dx)
    assert rel(dx, 2 * xt.grad.numpy()) <= 1e-12


def test_optimizer_family(orc):
    """Momentum / NAG / RMSprop / Adagrad against torch.optim (same update rules at constant learning rate);
    AdamW and AMSGrad against the reference's formulas written out in numpy (torch orders the decay and the
    bias correction of the running maximum differently)."""
    rng = np.random.default_rng(3)
    n, lr = 257, 0.01
    w0 = rng.standard_normal(n)
    grads = [rng.standard_normal(n) for _ in range(4)]
    ops = orc.Ops()

    def run_oracle(kind, h, nstate):
        w = w0.copy()
        s = [np.zeros(n) for _ in range(nstate)] + [None] * (3 - nstate)
        for t, g in enumerate(grads, 1):
            ops.optimizer_step(kind, w, g, s[0], s[1], s[2], lr, h, t)
        return w

    def run_torch(make):
        p = torch.nn.Parameter(torch.tensor(w0))
        opt = make([p])
        for g in grads:
            p.grad = torch.tensor(g)
            opt.step()
        return p.detach().numpy()

    assert rel(run_oracle(1, (0.9,), 1), run_torch(lambda p: torch.optim.SGD(p, lr=lr, momentum=0.9))) <= TOL
    assert rel(run_oracle(2, (0.9,), 1), run_torch(lambda p: torch.optim.SGD(p, lr=lr, momentum=0.9, nesterov=True))) <= TOL
    assert rel(run_oracle(3, (0.9, 1e-8), 1), run_torch(lambda p: torch.optim.RMSprop(p, lr=lr, alpha=0.9, eps=1e-8))) <= TOL
    assert rel(run_oracle(4, (0.0, 1e-8), 1), run_torch(lambda p: torch.optim.Adagrad(p, lr=lr, eps=1e-8))) <= TOL

    b1, b2, eps, wd = 0.9, 0.999, 1e-8, 0.01
    w, m, v, vmax = w0.copy(), np.zeros(n), np.zeros(n), np.zeros(n)
    w2 = w0.copy()
    for t, g in enumerate(grads, 1):
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        w = w - lr * (m / (1 - b1 ** t)) / (np.sqrt(v / (1 - b2 ** t)) + eps)
        w = w - lr * wd * w
        vmax = np.maximum(vmax, v)
        w2 = w2 - lr * (m / (1 - b1 ** t)) / (np.sqrt(vmax) + eps)
    assert rel(run_oracle(6, (b1, b2, eps, wd), 2), w) <= TOL
    assert rel(run_oracle(7, (b1, b2, eps), 3), w2) <= TOL


def test_vector_form_tape_ops(orc):
    """matVecMul, concatenate, elementWiseMultiply, sum and the parameterised activations on the oracle's tape
    against torch autograd: one LSTM-style step written in the reference's vector vocabulary."""
    rng = np.random.default_rng(21)
    H, I = 7, 5
    W1, W2, b, h0, x = (rng.standard_normal(s) for s in ((H, H + I), (H, H + I), (H,), (H,), (I,)))
    E = orc.Engine()
    oW1, oW2, ob, oh, ox = (orc.T(a) for a in (W1, W2, b, h0, x))
    z = E.concatenate(oh, ox)
    g1 = E.sigmoidMatrix(E.addMatrix(E.matVecMul(oW1, z), ob))
    g2 = E.act2(7, E.matVecMul(oW2, z))
    out = E.sum(E.elementWiseMultiply(E.elementWiseMultiply(g1, g2), oh))
    out.backward()
    tW1, tW2, tb, th, tx = (tt(a) for a in (W1, W2, b, h0, x))
    tz = torch.cat([th, tx])
    tout = (torch.sigmoid(tW1 @ tz + tb) * torch.nn.functional.silu(tW2 @ tz) * th).sum()
    tout.backward()
    assert abs(float(out.value) - float(tout)) <= 1e-12 * abs(float(tout))
    for o, t in ((oW1, tW1), (oW2, tW2), (ob, tb), (oh, th), (ox, tx)):
        assert rel(o.grad, t.grad.numpy()) <= TOL


@pytest.mark.parametrize("padding,kh", [("valid", 3), ("same", 3), ("same", 5), ("valid", 1), ("same", 4)])
def test_conv2d(orc, padding, kh):
    """conv2d (tensor.dart:765-833) against torch's cross-correlation; 'same' with an even kernel pads (k-1)//2 on
    every side like the reference, so the output shrinks by one."""
    rng = np.random.default_rng(kh)
    x, k, bias = rng.standard_normal((9, 11)), rng.standard_normal((kh, kh)), rng.standard_normal(())
    E = orc.Engine()
    ox, ok, ob = orc.T(x), orc.T(k), orc.T(bias)
    out = E.addScalarToMatrix(E.conv2d(ox, ok, padding), ob)
    loss = E.mseMatrix(out, orc.T(np.zeros_like(out.value)))
    loss.backward()
    tx, tk, tb = tt(x), tt(k), tt(bias)
    pad = (kh - 1) // 2 if padding == "same" else 0
    tout = torch.nn.functional.conv2d(tx[None, None], tk[None, None], padding=pad)[0, 0] + tb
    (tout ** 2).mean().backward()
    assert rel(out.value, tout.detach().numpy()) <= TOL
    for o, t in ((ox, tx), (ok, tk), (ob, tb)):
        assert rel(o.grad, t.grad.numpy()) <= TOL
