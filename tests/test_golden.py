"""The committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py) against the
oracle on CPU and against the CUDA path on the GPU."""
import os

import numpy as np
import pytest

from tests.gpu_util import TOL_TF32, rel

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
w64 = lambda x: np.ascontiguousarray(x, dtype=np.float64)  # noqa: E731


def load(name):
    return dict(np.load(os.path.join(G, name)))


def test_oracle_reproduces_goldens(orc):
    g = load("gemm_gelu_48x32x40.npz")
    o = orc.gemm_gelu_fwd_bwd(w64(g["A"]), w64(g["B"]), w64(g["bias"]), w64(g["dC"]))
    for k in ("Z", "C", "dZ", "dA", "dB", "dbias"):
        assert np.array_equal(o[k], g[k]), k
    m = load("mlp_32_16_12_5.npz")
    o = orc.mlp_step(w64(m["X"]), m["labels"], [w64(m[f"p{i}"]) for i in range(6)], lr=0.01)
    assert np.array_equal(o["logits"], m["logits"]) and o["loss"] == float(m["loss"])
    for i in range(6):
        assert np.array_equal(o["grads"][i], m[f"g{i}"]) and np.array_equal(o["params"][i], m[f"n{i}"])
    s = load("lstm_T5_B3_I8_H12.npz")
    h, loss, dW, db = orc.Ops().lstm_fwd_bwd(w64(s["W"]), w64(s["b"]), w64(s["x"]), w64(s["target"]))
    assert np.array_equal(h, s["h_last"]) and loss == float(s["loss"]) and np.array_equal(dW, s["dW"])
    r = load("rows_6x16.npz")
    assert np.array_equal(orc.Ops().softmax_fwd(w64(r["x"]), 6), r["softmax_causal"])


def test_oracle_reproduces_widened_goldens(orc):
    g = load("widened_ops.npz")
    ops = orc.Ops()
    for kind, h, nstate in ((1, (0.9,), 1), (2, (0.9,), 1), (3, (0.9, 1e-8), 1), (4, (0.0, 1e-8), 1),
                            (6, (0.9, 0.999, 1e-8, 0.01), 2), (7, (0.9, 0.999, 1e-8), 3)):
        w = w64(g["opt_w0"])
        st = [np.zeros(w.size) for _ in range(nstate)] + [None] * (3 - nstate)
        for t, gr in enumerate(g["opt_grads"], 1):
            ops.optimizer_step(kind, w, w64(gr), st[0], st[1], st[2], 0.01, h, t)
        assert np.array_equal(w, g[f"opt_w_kind{kind}"]), kind
    for kind, alpha in ((5, 0.01), (6, 1.0), (7, 0.0), (8, 0.0)):
        assert np.array_equal(ops.act2_fwd(kind, alpha, w64(g["act_x"])), g[f"act_y_kind{kind}"])
    assert np.array_equal(ops.conv2d_fwd(w64(g["conv_x"]), w64(g["conv_k"]), 1), g["conv_out"])


@pytest.mark.gpu
def test_gpu_matches_widened_goldens():
    """Optimizer rules, parameterised activations, conv2d and one fused-attention head against the committed vectors."""
    import ctypes as C
    from flutter_ml_b200 import _lib
    g = load("widened_ops.npz")
    ctx = _lib.Context(precision=_lib.PREC_TF32)
    n = g["opt_w0"].size
    for kind, h, nstate in ((1, (0.9,), 1), (2, (0.9,), 1), (3, (0.9, 1e-8), 1), (4, (0.0, 1e-8), 1),
                            (6, (0.9, 0.999, 1e-8, 0.01), 2), (7, (0.9, 0.999, 1e-8), 3)):
        w = ctx.upload(g["opt_w0"])
        st = [ctx.zeros(n) for _ in range(nstate)] + [None] * (3 - nstate)
        hh = tuple(h) + (0.0,) * (4 - len(h))
        for t, gr in enumerate(g["opt_grads"], 1):
            ctx.call("fml_optimizer_step", kind, w, ctx.upload(gr), st[0], st[1], st[2], n, 0.01, *hh, t)
        assert rel(w.numpy(), g[f"opt_w_kind{kind}"]) <= 1e-6, kind
    x, dy = ctx.upload(g["act_x"]), ctx.upload(g["act_dy"])
    for kind, alpha in ((5, 0.01), (6, 1.0), (7, 0.0), (8, 0.0)):
        y, dx = ctx.empty(64), ctx.empty(64)
        ctx.call("fml_act2_fwd", kind, alpha, x, y, 64)
        ctx.call("fml_act2_bwd", kind, alpha, x, dy, dx, 64, 0)
        assert rel(y.numpy(), g[f"act_y_kind{kind}"]) <= 1e-6 and rel(dx.numpy(), g[f"act_dx_kind{kind}"]) <= 1e-6
    img, ker, dout = ctx.upload(g["conv_x"]), ctx.upload(g["conv_k"]), ctx.upload(g["conv_dout"])
    out, dimg, dker = ctx.empty(9, 11), ctx.zeros(9, 11), ctx.zeros(3, 3)
    ctx.call("fml_conv2d_fwd", img, ker, None, out, 1, 9, 11, 1, 3, 3, 1)
    ctx.call("fml_conv2d_bwd", img, ker, dout, dimg, dker, None, 1, 9, 11, 1, 3, 3, 1, launches=2)
    assert rel(out.numpy(), g["conv_out"]) <= 1e-6 and rel(dimg.numpy(), g["conv_dx"]) <= 1e-6 and rel(dker.numpy(), g["conv_dk"]) <= 1e-6
    S, dk = g["att_q"].shape
    qkv = ctx.upload(np.concatenate([g["att_q"], g["att_k"], g["att_v"]], axis=1))
    o, lse, G_, dqkv, scratch = ctx.empty(S, dk), ctx.empty(S), ctx.upload(g["att_g"]), ctx.empty(S, 3 * dk), ctx.empty(S)
    d = _lib.AttentionDesc()
    d.n_seq, d.seq_len, d.heads, d.d_head = 1, S, 1, dk
    d.q, d.k, d.v, d.ld_qkv, d.out, d.ld_out, d.lse, d.scale, d.causal = qkv.ptr, qkv.ptr + 4 * dk, qkv.ptr + 8 * dk, 3 * dk, o.ptr, dk, lse.ptr, 0.125, 1
    ctx.check(ctx.lib.fml_attention_fwd(ctx.h, C.byref(d)))
    ctx.check(ctx.lib.fml_attention_bwd(ctx.h, C.byref(d), G_.ptr, dk, dqkv.ptr, dqkv.ptr + 4 * dk, dqkv.ptr + 8 * dk, 3 * dk, 0, scratch.ptr))
    assert rel(o.numpy(), g["att_out"]) <= 2e-3
    got = dqkv.numpy()
    for i, name in enumerate(("att_dq", "att_dk", "att_dv")):
        assert rel(got[:, i * dk:(i + 1) * dk], g[name]) <= 5e-3, name
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.gpu
def test_gpu_matches_goldens():
    from flutter_ml_b200 import _lib, models, ops
    ctx = _lib.Context()
    g = load("gemm_gelu_48x32x40.npz")
    M, K = g["A"].shape
    N = g["B"].shape[1]
    d = {k: ctx.upload(g[k]) for k in ("A", "B", "bias", "dC")}
    C, Z, dZ, dA, dB, db = ctx.empty(M, N), ctx.empty(M, N), ctx.empty(M, N), ctx.empty(M, K), ctx.empty(K, N), ctx.zeros(N)
    ops.dense_forward(ctx, d["A"], d["B"], d["bias"], "gelu", M, N, K, C, Z)
    ops.dense_backward(ctx, d["A"], d["B"], Z, d["dC"], "gelu", M, N, K, dZ, dA, dB, db)
    for name, got in (("C", C), ("Z", Z), ("dZ", dZ), ("dA", dA), ("dB", dB), ("dbias", db)):
        assert rel(got.numpy(), g[name]) <= 2 * TOL_TF32, name
    r = load("rows_6x16.npz")
    x, y = ctx.upload(r["x"]), ctx.empty(6, 16)
    ctx.call("fml_softmax_rows_fwd", x, y, 6, 16, 1.0, 6)
    assert rel(y.numpy(), r["softmax_causal"]) <= 1e-6
    gm, be = ctx.upload(r["gamma"]), ctx.upload(r["beta"])
    ly, xh, rs = ctx.empty(6, 16), ctx.empty(6, 16), ctx.empty(6)
    ctx.call("fml_layernorm_fwd", x, None, gm, be, ly, xh, rs, 6, 16, 1e-5)
    assert rel(ly.numpy(), r["ln_y"]) <= 2e-6
    m = load("mlp_32_16_12_5.npz")
    mlp = models.MLP(ctx, [m[f"p{i}"] for i in range(6)], lr=0.01, precision=_lib.PREC_FP32)
    loss, logits, grads = mlp.train_step(ctx.upload(m["X"]), ctx.upload(m["labels"]), keep=True)
    assert rel(logits.numpy(), m["logits"]) <= 1e-5 and abs(loss.numpy()[0] - float(m["loss"])) <= 1e-5
    ctx.close()
