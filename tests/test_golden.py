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
