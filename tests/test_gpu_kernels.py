"""Parity of every CUDA kernel against the float64 oracle, through the C ABI."""
import numpy as np
import pytest

from tests.gpu_util import TOL_3XTF32, TOL_FP32, TOL_TF32, ctx, rel  # noqa: F401

pytestmark = pytest.mark.gpu
f64 = np.float64


def w64(x):
    return np.ascontiguousarray(x, dtype=np.float64)


GEMM_CASES = [
    # M, N, K, transA, transB
    (128, 256, 32, 0, 1), (128, 256, 128, 0, 0), (128, 256, 128, 1, 0), (128, 256, 128, 1, 1),
    (300, 200, 100, 0, 0), (300, 200, 100, 1, 0), (300, 200, 100, 0, 1), (77, 64, 40, 1, 1),
    (1, 4, 4, 0, 0), (513, 1028, 260, 0, 0), (64, 784, 128, 0, 1), (64, 10, 64, 0, 0), (784, 128, 64, 1, 0),
    (1024, 1024, 1024, 0, 0), (2048, 512, 4096, 1, 0),
]


@pytest.mark.parametrize("prec,tol", [(0, TOL_TF32), (1, TOL_3XTF32), (2, TOL_FP32)])
@pytest.mark.parametrize("M,N,K,tA,tB", GEMM_CASES)
def test_gemm_matches_oracle(ctx, orc, M, N, K, tA, tB, prec, tol):
    rng = np.random.default_rng(M + 3 * N + 7 * K + tA + 2 * tB)
    A = (rng.standard_normal((K, M) if tA else (M, K)) / np.sqrt(K)).astype(np.float32)
    B = (rng.standard_normal((N, K) if tB else (K, N)) / np.sqrt(K)).astype(np.float32)
    dA, dB, dC = ctx.upload(A), ctx.upload(B), ctx.empty(M, N)
    ctx.gemm(dA, dB, dC, M, N, K, transA=bool(tA), transB=bool(tB), precision=prec)
    ops = orc.Ops(omp=True)
    opA = w64(A.T if tA else A)
    opB = w64(B.T if tB else B)
    ref = ops.matmul_fwd(opA, opB)
    assert rel(dC.numpy(), ref) <= tol
    for a in (dA, dB, dC):
        a.free()


@pytest.mark.parametrize("beta", [0.0, 1.0])
@pytest.mark.parametrize("M,N,K,tA,tB,prec", [(64, 10, 16384, 1, 0, 0), (64, 10, 16384, 1, 0, 2), (100, 30, 5000, 0, 1, 2),
                                             (10, 64, 4099, 0, 0, 2)])
def test_cuda_core_gemm_with_k_slices(ctx, orc, M, N, K, tA, tB, prec, beta):
    """A few output tiles under a long k on the CUDA-core path (a 10-wide head's weight gradient over a 16384-row
    batch: leading dimension 10 keeps it off the tensor-core path): k is cut into slices that are summed with
    atomics; beta 0 starts from a zeroed C, beta 1 adds to what is there."""
    rng = np.random.default_rng(M + N + K)
    A = (rng.standard_normal((K, M) if tA else (M, K)) / np.sqrt(K)).astype(np.float32)
    B = (rng.standard_normal((N, K) if tB else (K, N)) / np.sqrt(K)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    dA, dB, dC = ctx.upload(A), ctx.upload(B), ctx.upload(C0)
    ctx.gemm(dA, dB, dC, M, N, K, transA=bool(tA), transB=bool(tB), precision=prec, alpha=0.5, beta=beta)
    assert ctx.gemm_last_path() == 2
    ref = 0.5 * orc.Ops(omp=True).matmul_fwd(w64(A.T if tA else A), w64(B.T if tB else B)) + beta * w64(C0)
    assert rel(dC.numpy(), ref) <= TOL_FP32
    for a in (dA, dB, dC):
        a.free()


def test_all_ones_1024_known_answer(ctx):
    # lib/gpu_benching.dart:34-37,60: all-ones 1024^3 => every element equals k (exact in TF32)
    n = 1024
    ones = np.ones((n, n), dtype=np.float32)
    dA, dB, dC = ctx.upload(ones), ctx.upload(ones), ctx.empty(n, n)
    ctx.gemm(dA, dB, dC, n, n, n)
    assert ctx.gemm_last_path() == 1
    assert np.all(dC.numpy() == float(n))


def test_legacy_multiply_matrices(ctx):
    # cuda_lib/kernel.cu:6-11 signature with host pointers; lib/gpu_benching.dart's check
    m, k, n = 33, 50, 21
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32)
    c = np.zeros((m, n), dtype=np.float32)
    ctx.lib.multiplyMatrices(a.ctypes.data, b.ctypes.data, c.ctypes.data, m, k, n)
    assert rel(c, w64(a) @ w64(b)) <= TOL_TF32


@pytest.mark.parametrize("act", ["relu", "sigmoid", "tanh", "gelu"])
@pytest.mark.parametrize("prec,tol", [(0, TOL_TF32), (1, TOL_3XTF32), (2, TOL_FP32)])
def test_dense_forward_backward(ctx, orc, act, prec, tol):
    """act(X.W+b) and its three gradients: the fused epilogue, the dZ kernel with column sums,
    dX = dZ.W^T and dW = X^T.dZ (tensor.dart:867-947, 679-709, 1013-1038).

    Each kernel is held to the tolerance on ITS OWN inputs: the gate of ReLU is discontinuous,
    so a pre-activation that differs from the oracle's in the last TF32 bit may flip it; the
    activation-gradient kernel is therefore checked against the oracle formula evaluated on the
    pre-activation the GPU produced, and the two backward products against the oracle products
    of the GPU's dZ."""
    M, K, N = 200, 96, 136
    rng = np.random.default_rng(11)
    X = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    dY = rng.standard_normal((M, N)).astype(np.float32)
    E = orc.Engine(omp=True)
    x, w, bt = orc.T(w64(X)), orc.T(w64(W)), orc.T(w64(b))
    y = E.dense_matrix(x, w, bt, act)
    z = y.inputs[0]
    dX_, dW_, db_, Y_, Z_ = ctx.empty(M, K), ctx.empty(K, N), ctx.zeros(N), ctx.empty(M, N), ctx.empty(M, N)
    dXd, dWd, bd, dYd = ctx.upload(X), ctx.upload(W), ctx.upload(b), ctx.upload(dY)
    dZ = ctx.empty(M, N)
    ctx.gemm(dXd, dWd, Y_, M, N, K, bias=bd, preact=Z_, act=act, precision=prec)
    saved = Z_ if act in ("relu", "gelu") else Y_
    ctx.call("fml_act_bwd", _act(act), saved, dYd, dZ, M, N, 0, db_)
    ctx.gemm(dZ, dWd, dX_, M, K, N, transB=True, precision=prec)
    ctx.gemm(dXd, dZ, dW_, K, N, M, transA=True, precision=prec)
    assert rel(Y_.numpy(), y.value) <= tol
    assert rel(Z_.numpy(), z.value) <= tol
    # activation gradient on the GPU's own saved tensor
    saved_h, dZ_h = w64(saved.numpy()), w64(dZ.numpy())
    dz_ref = np.zeros((M, N))
    E.ops.unary_bwd(act, saved_h, w64(dY), dz_ref)
    assert rel(dZ_h, dz_ref) <= 2e-6
    assert rel(db_.numpy(), dZ_h.sum(0)) <= 2e-6
    if act != "relu":  # smooth activations: the whole chain also stays within the tolerance
        y.grad = w64(dY)
        for node in (y, z, z.inputs[0]):
            node.backward_fn()
        assert rel(dZ_h, z.grad) <= tol
        assert rel(db_.numpy(), bt.grad) <= tol * 2
        assert rel(dX_.numpy(), x.grad) <= tol * 2
        assert rel(dW_.numpy(), w.grad) <= tol * 2
    # backward products against the oracle products of the same dZ (tensor.dart:918-924, 935-941)
    dx_ref, dw_ref = np.zeros((M, K)), np.zeros((K, N))
    E.ops.matmul_bwd(w64(X), w64(W), dZ_h, dx_ref, dw_ref)
    assert rel(dX_.numpy(), dx_ref) <= tol
    assert rel(dW_.numpy(), dw_ref) <= tol


def _act(name):
    from flutter_ml_b200 import _lib
    return _lib.ACT_BY_NAME[name]


def test_gemm_accumulates_with_beta(ctx):
    M, N, K = 130, 72, 64
    rng = np.random.default_rng(5)
    A, B, C0 = [rng.standard_normal(s).astype(np.float32) for s in ((M, K), (K, N), (M, N))]
    dA, dB, dC = ctx.upload(A), ctx.upload(B), ctx.upload(C0)
    ctx.gemm(dA, dB, dC, M, N, K, beta=1.0)
    assert rel(dC.numpy(), w64(C0) + w64(A) @ w64(B)) <= TOL_TF32


@pytest.mark.parametrize("prec,tol", [(0, TOL_TF32), (2, TOL_FP32)])
def test_batched_strided_attention_products(ctx, prec, tol):
    """QK^T and P.V per (sequence, head) straight out of a fused [B*S, 3d] projection
    (lib/layertypes/singleHeadAttentionLayer.dart:77-86)."""
    Bn, H, S, dk = 3, 4, 96, 64
    d = H * dk
    rng = np.random.default_rng(9)
    qkv = rng.standard_normal((Bn * S, 3 * d)).astype(np.float32)
    dq = ctx.upload(qkv)
    scores = ctx.empty(Bn, H, S, S)
    ctx.gemm(dq, dq.view(d, ()), scores, S, S, dk, transB=True, lda=3 * d, ldb=3 * d, ldc=S, batch=(H, Bn),
             sA=(dk, S * 3 * d), sB=(dk, S * 3 * d), sC=(S * S, H * S * S), alpha=0.125, precision=prec)
    q = w64(qkv).reshape(Bn, S, 3, H, dk)
    ref = np.einsum("bshd,bthd->bhst", q[:, :, 0], q[:, :, 1]) * 0.125
    assert rel(scores.numpy(), ref) <= tol
    out = ctx.empty(Bn * S, d)
    ctx.gemm(scores, dq.view(2 * d, ()), out, S, dk, S, lda=S, ldb=3 * d, ldc=d, batch=(H, Bn),
             sA=(S * S, H * S * S), sB=(dk, S * 3 * d), sC=(dk, S * d), precision=prec)
    # P.V is checked on the scores the GPU produced (one product per tolerance)
    ref2 = np.einsum("bhst,bthd->bshd", w64(scores.numpy()), q[:, :, 2]).reshape(Bn * S, d)
    assert rel(out.numpy(), ref2) <= tol


@pytest.mark.parametrize("rows,cols,causal", [(64, 10, 0), (96 * 3, 96, 96), (500, 256, 0), (33, 1000, 0),
                                              (40, 2048, 0), (7, 4100, 0), (512, 512, 512)])
def test_softmax_rows(ctx, orc, rows, cols, causal):
    rng = np.random.default_rng(rows + cols)
    x = (3 * rng.standard_normal((rows, cols))).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    scale = 0.125
    ops = orc.Ops()
    y_ref = ops.softmax_fwd(w64(x) * scale, causal)
    dx_ref = np.zeros((rows, cols))
    ops.softmax_bwd(y_ref, w64(dy), dx_ref)
    dx_ref *= scale
    dxx, dyy, y, dx = ctx.upload(x), ctx.upload(dy), ctx.empty(rows, cols), ctx.empty(rows, cols)
    ctx.call("fml_softmax_rows_fwd", dxx, y, rows, cols, scale, causal)
    ctx.call("fml_softmax_rows_bwd", y, dyy, dx, rows, cols, scale, 0)
    yh = y.numpy()
    assert rel(yh, y_ref) <= 1e-6
    if causal:
        r = np.arange(rows)[:, None] % causal
        assert np.all(yh[np.arange(cols)[None, :] > r] == 0.0)
    assert rel(dx.numpy(), dx_ref) <= 2e-6


@pytest.mark.parametrize("rows,cols,res", [(100, 512, True), (37, 1024, False), (64, 96, True), (20, 1030, True),
                                           (300, 2048, False), (5, 16, True)])
def test_layernorm(ctx, orc, rows, cols, res):
    rng = np.random.default_rng(rows * cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    r = rng.standard_normal((rows, cols)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    b = (0.1 * rng.standard_normal(cols)).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    ops = orc.Ops()
    xin = w64(x) + (w64(r) if res else 0)
    y_ref, xhat_ref, var_ref = ops.layernorm_fwd(xin, w64(g), w64(b))
    dx_ref, dg_ref, db_ref = np.zeros((rows, cols)), np.zeros(cols), np.zeros(cols)
    ops.layernorm_bwd(w64(dy), w64(g), xhat_ref, var_ref, dx_ref, dg_ref, db_ref)
    dxx, dr, dg, db_, ddy = ctx.upload(x), ctx.upload(r), ctx.upload(g), ctx.upload(b), ctx.upload(dy)
    y, xhat, rstd = ctx.empty(rows, cols), ctx.empty(rows, cols), ctx.empty(rows)
    dx, dgam, dbet = ctx.empty(rows, cols), ctx.zeros(cols), ctx.zeros(cols)
    ctx.call("fml_layernorm_fwd", dxx, dr if res else None, dg, db_, y, xhat, rstd, rows, cols, 1e-5)
    ctx.call("fml_layernorm_bwd", ddy, dg, xhat, rstd, dx, dgam, dbet, rows, cols, 0)
    assert rel(y.numpy(), y_ref) <= 2e-6
    assert rel(xhat.numpy(), xhat_ref) <= 2e-6
    assert rel(dx.numpy(), dx_ref) <= 1e-5
    assert rel(dgam.numpy(), dg_ref) <= 1e-5 and rel(dbet.numpy(), db_ref) <= 1e-5


@pytest.mark.parametrize("rows,cols", [(64, 10), (200, 1000), (16, 32000), (301, 4100), (40, 12288), (9, 32768)])
def test_softmax_xent(ctx, orc, rows, cols):
    rng = np.random.default_rng(cols)
    z = (2 * rng.standard_normal((rows, cols))).astype(np.float32)
    labels = rng.integers(0, cols, rows).astype(np.int32)
    inv = 1.0 / (3 * rows)
    dz_ref = np.zeros((rows, cols))
    loss_ref = orc.Ops().softmax_xent(w64(z), labels, dz_ref, inv)
    dzz, dl, loss = ctx.upload(z), ctx.upload(labels), ctx.zeros(1)
    ctx.call("fml_softmax_xent", dzz, dl, dzz, loss, rows, cols, inv, launches=2)  # in place
    assert abs(loss.numpy()[0] - loss_ref) <= 2e-6 * abs(loss_ref)
    assert rel(dzz.numpy(), dz_ref) <= 2e-6


@pytest.mark.parametrize("rows,cols", [(64, 10), (301, 4100), (700, 12288), (40, 32768)])
def test_softmax_xent_with_bias_gradient(ctx, orc, rows, cols):
    """fml_softmax_xent_dbias: loss and gradient as fml_softmax_xent, plus the column sums of the gradient ADDED into
    dbias (addMatrixAndVector backward, tensor.dart:698-704) by the same pass."""
    rng = np.random.default_rng(cols + 1)
    z = (2 * rng.standard_normal((rows, cols))).astype(np.float32)
    labels = rng.integers(0, cols, rows).astype(np.int32)
    inv = 1.0 / rows
    dz_ref = np.zeros((rows, cols))
    loss_ref = orc.Ops().softmax_xent(w64(z), labels, dz_ref, inv)
    base = rng.standard_normal(cols).astype(np.float32)
    dzz, dl, loss, db = ctx.upload(z), ctx.upload(labels), ctx.zeros(1), ctx.upload(base)
    ctx.call("fml_softmax_xent_dbias", dzz, dl, dzz, loss, rows, cols, inv, db, launches=3)
    assert abs(loss.numpy()[0] - loss_ref) <= 2e-6 * abs(loss_ref)
    assert rel(dzz.numpy(), dz_ref) <= 2e-6
    got = db.numpy().astype(np.float64) - base
    # fp32: one rounding of base + sum per column, plus the summation error of the column sums themselves
    assert np.linalg.norm(got - dz_ref.sum(0)) <= 2e-7 * np.linalg.norm(base) + 1e-5 * np.linalg.norm(dz_ref.sum(0))


def test_mse(ctx, orc):
    rng = np.random.default_rng(3)
    p, t = rng.standard_normal((257, 129)).astype(np.float32), rng.standard_normal((257, 129)).astype(np.float32)
    ops = orc.Ops()
    dp_ref = np.zeros(p.shape)
    ops.mse_bwd(w64(p), w64(t), dp_ref, 1.0)
    dpp, dt, dp, loss = ctx.upload(p), ctx.upload(t), ctx.empty(*p.shape), ctx.zeros(1)
    ctx.call("fml_mse", dpp, dt, dp, loss, p.size, 1.0, launches=2)
    assert abs(loss.numpy()[0] - ops.mse_fwd(w64(p), w64(t))) <= 1e-6
    assert rel(dp.numpy(), dp_ref) <= 1e-6


@pytest.mark.parametrize("n", [109386, 4096, 7])
def test_sgd_and_adam(ctx, orc, n):
    rng = np.random.default_rng(n)
    w, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    ops = orc.Ops()
    w_ref = w64(w)
    ops.sgd_step(w_ref, w64(g), 0.01)
    dw, dg = ctx.upload(w), ctx.upload(g)
    ctx.call("fml_sgd_step", dw, dg, n, 0.01, 1.0)
    assert rel(dw.numpy(), w_ref) <= 1e-7
    w_ref, m_ref, v_ref = w64(w), np.zeros(n), np.zeros(n)
    dw, dm, dv = ctx.upload(w), ctx.zeros(n), ctx.zeros(n)
    for t in (1, 2, 3):
        ops.adam_step(w_ref, w64(g), m_ref, v_ref, 1e-3, t)
        ctx.call("fml_adam_step", dw, dg, dm, dv, n, 1e-3, 0.9, 0.999, 1e-8, t, 1.0)
    assert rel(dw.numpy(), w_ref) <= 1e-6
    assert rel(dm.numpy(), m_ref) <= 1e-6 and rel(dv.numpy(), v_ref) <= 1e-6


def test_embedding_and_positional(ctx, orc):
    V, d, S, Bn = 50, 64, 12, 3
    rng = np.random.default_rng(8)
    table = rng.standard_normal((V, d)).astype(np.float32)
    ids = rng.integers(0, V, Bn * S).astype(np.int32)
    dout = rng.standard_normal((Bn * S, d)).astype(np.float32)
    ops = orc.Ops()
    pe_ref = ops.positional_table(S, d)
    out_ref = ops.embedding_fwd(w64(table), ids) + np.tile(pe_ref, (Bn, 1))
    dt_ref = np.zeros((V, d))
    ops.embedding_bwd(w64(dout), ids, dt_ref)
    dtab, dids, pe, out, ddout, dtable = (ctx.upload(table), ctx.upload(ids), ctx.empty(S, d), ctx.empty(Bn * S, d),
                                          ctx.upload(dout), ctx.zeros(V, d))
    ctx.call("fml_positional_table", pe, S, d)
    ctx.call("fml_embedding_fwd", dtab, dids, pe, out, Bn * S, d, S, V)
    ctx.call("fml_embedding_bwd", ddout, dids, dtable, Bn * S, d, V)
    assert rel(pe.numpy(), pe_ref) <= 1e-7
    assert rel(out.numpy(), out_ref) <= 1e-7
    assert rel(dtable.numpy(), dt_ref) <= 1e-6


def test_small_elementwise(ctx):
    rng = np.random.default_rng(2)
    a, b = rng.standard_normal((67, 45)).astype(np.float32), rng.standard_normal((67, 45)).astype(np.float32)
    da, db_, y = ctx.upload(a), ctx.upload(b), ctx.empty(67, 45)
    ctx.call("fml_add", da, db_, y, a.size)
    assert np.array_equal(y.numpy(), a + b)
    ctx.call("fml_mul", da, db_, y, a.size)
    assert np.array_equal(y.numpy(), a * b)
    ctx.call("fml_axpy", 0.5, da, y, a.size)
    assert np.allclose(y.numpy(), a * b + 0.5 * a, rtol=1e-6, atol=1e-6)
    t = ctx.empty(45, 67)
    ctx.call("fml_transpose", da, t, 67, 45)
    assert np.array_equal(t.numpy(), a.T)
    cs = ctx.empty(45)
    ctx.call("fml_col_sum", da, cs, 67, 45, 0)
    assert rel(cs.numpy(), a.astype(np.float64).sum(0)) <= 1e-6
    bias = ctx.upload(b[0])
    ctx.call("fml_add_bias", da, bias, y, 67, 45)
    assert np.array_equal(y.numpy(), a + b[0][None, :])


@pytest.mark.parametrize("prec,tol", [(0, TOL_TF32), (1, 2e-5), (2, 2e-5)])
def test_lstm_forward_backward(orc, prec, tol):
    """LSTMLayer (lib/layertypes/lstmLayer.dart:112-150) + mse on the last hidden state, BPTT."""
    from flutter_ml_b200 import _lib
    c = _lib.Context(precision=prec)
    T, B, I, H = 12, 20, 24, 32
    rng = np.random.default_rng(13)
    a = 1 / np.sqrt(H)
    W = rng.uniform(-a, a, (4, H, H + I)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (4, H)).astype(np.float32)
    x = rng.standard_normal((B, T, I)).astype(np.float32)
    target = rng.standard_normal((B, H)).astype(np.float32)
    h_ref, loss_ref, dW_ref, db_ref = orc.Ops(omp=True).lstm_fwd_bwd(w64(W), w64(b), w64(x), w64(target))
    dW_, db_, dx_ = c.zeros(4 * H, H + I), c.zeros(4 * H), c.empty(T * B, I)
    d = _lib.LstmDesc()
    d.T, d.B, d.I, d.H = T, B, I, H
    bufs = dict(W=c.upload(W), b=c.upload(b), x=c.upload(np.ascontiguousarray(x.transpose(1, 0, 2))),
                gates=c.empty(T, B, 4 * H), cells=c.empty(T + 1, B, H), hs=c.empty(T + 1, B, H), xproj=c.empty(T * B, 4 * H))
    for k, v in bufs.items():
        setattr(d, k, v.ptr)
    import ctypes
    c.check(c.lib.fml_lstm_fwd(c.h, ctypes.byref(d)))
    h_last = bufs["hs"].view(T * B * H, (B, H))
    # loss = sum over sequences of mse(h_T, target): dh = 2 (h - t) / H
    dh, loss = c.empty(B, H), c.zeros(1)
    c.call("fml_mse", h_last, c.upload(target), dh, loss, B * H, float(B))
    scratch = c.empty(T * B * 4 * H + 2 * B * H)
    c.check(c.lib.fml_lstm_bwd(c.h, ctypes.byref(d), dh.ptr, dW_.ptr, db_.ptr, dx_.ptr, scratch.ptr))
    assert c.device_status() == 0
    assert rel(h_last.numpy(), h_ref) <= tol
    assert abs(loss.numpy()[0] * B - loss_ref) <= tol * abs(loss_ref) * 4
    assert rel(dW_.numpy().reshape(4, H, H + I), dW_ref) <= tol * 2
    assert rel(db_.numpy().reshape(4, H), db_ref) <= tol * 2
    c.close()


@pytest.mark.parametrize("T,B,I,H", [(6, 128, 16, 256), (5, 70, 8, 320), (9, 3, 4, 64), (3, 16, 8, 1024), (1, 5, 4, 32)])
def test_lstm_single_kernel_forward_recurrence(orc, T, B, I, H):
    """The cooperative forward kernel (TF32 mode, batch <= 128) on shapes that exercise a full 128-row batch, a TMA ring
    that wraps (H = 320: 10 k-blocks through 8 stages) and a nearly empty batch: every h_t, c_t and saved gate against
    the oracle's step-by-step recurrence (lstmLayer.dart:112-150)."""
    import ctypes
    from flutter_ml_b200 import _lib
    c = _lib.Context(precision=_lib.PREC_TF32)
    rng = np.random.default_rng(T * 1000 + H)
    a = 1 / np.sqrt(H)
    W = rng.uniform(-a, a, (4, H, H + I)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (4, H)).astype(np.float32)
    x = rng.standard_normal((T, B, I)).astype(np.float32)
    d = _lib.LstmDesc()
    d.T, d.B, d.I, d.H = T, B, I, H
    bufs = dict(W=c.upload(W), b=c.upload(b), x=c.upload(x), gates=c.empty(T, B, 4 * H), cells=c.empty(T + 1, B, H),
                hs=c.empty(T + 1, B, H), xproj=c.empty(T * B, 4 * H))
    for k, v in bufs.items():
        setattr(d, k, v.ptr)
    c.check(c.lib.fml_lstm_fwd(c.h, ctypes.byref(d)))
    assert c.device_status() == 0
    hs, cs, gates = bufs["hs"].numpy(), bufs["cells"].numpy(), bufs["gates"].numpy().reshape(T, B, H, 4)
    W64, b64 = w64(W), w64(b)
    h, cc = np.zeros((B, H)), np.zeros((B, H))
    sig = lambda z: 1 / (1 + np.exp(-z))
    for t in range(T):
        z = np.concatenate([h, w64(x[t])], axis=1)                     # [h_{t-1}, x_t] (lstmLayer.dart:119)
        f, i, g, o = (z @ W64[q].T + b64[q] for q in range(4))
        f, i, g, o = sig(f), sig(i), np.tanh(g), sig(o)
        cc = f * cc + i * g
        h = o * np.tanh(cc)
        assert rel(hs[t + 1], h) <= TOL_TF32 and rel(cs[t + 1], cc) <= TOL_TF32, t
        assert rel(gates[t], np.stack([f, i, g, o], axis=-1)) <= TOL_TF32, t
    assert np.all(hs[0] == 0)
    c.close()


@pytest.mark.parametrize("act", ["relu", "sigmoid", "tanh", "gelu"])
@pytest.mark.parametrize("prec", [0, 2])
def test_gemm_gradient_epilogue_equals_separate_kernel(ctx, act, prec):
    """fml_gemm with dact_saved: (dZ.W^T) * act'(saved) in the epilogue equals the product followed by fml_act_bwd
    (the dLoss/dAct multiply of tensor.dart:1030 / :552 / :598 applied to tensor.dart:918-924)."""
    M, N, K = 200, 136, 96
    rng = np.random.default_rng(21)
    dZ = rng.standard_normal((M, K)).astype(np.float32)
    W = rng.standard_normal((N, K)).astype(np.float32)
    saved = rng.standard_normal((M, N)).astype(np.float32)
    if act in ("sigmoid", "tanh"):
        saved = np.tanh(saved).astype(np.float32) * (0.5 if act == "sigmoid" else 1.0) + (0.5 if act == "sigmoid" else 0.0)
    d_dz, d_w, d_s = ctx.upload(dZ), ctx.upload(W), ctx.upload(saved)
    fused, plain, ref = ctx.empty(M, N), ctx.empty(M, N), ctx.empty(M, N)
    ctx.gemm(d_dz, d_w, fused, M, N, K, transB=True, precision=prec, dact_saved=d_s, dact=act)
    ctx.gemm(d_dz, d_w, plain, M, N, K, transB=True, precision=prec)
    ctx.call("fml_act_bwd", _act(act), d_s, plain, ref, M, N, 0, None)
    assert rel(fused.numpy(), ref.numpy()) <= 2e-6


@pytest.mark.parametrize("S,causal", [(64, True), (96, False), (256, True), (512, True), (512, False), (320, True)])
@pytest.mark.parametrize("prec,tol", [(0, TOL_TF32), (1, 2e-5)])
def test_attention_scores_with_row_epilogue(ctx, orc, S, causal, prec, tol):
    """fml_gemm rowop 1/2: Q.K^T with scale + causal mask + softmax in the epilogue, and dO.V^T with the softmax
    backward in the epilogue, against the oracle's matMul / scaleMatrix / softmaxMatrix chain
    (singleHeadAttentionLayer.dart:77-81, softmax.dart:68-115)."""
    Bn, H, dk = 2, 3, 64
    rng = np.random.default_rng(S + 7 * causal)
    Q, Kx = rng.standard_normal((Bn, H, S, dk)).astype(np.float32), rng.standard_normal((Bn, H, S, dk)).astype(np.float32)
    dPh = rng.standard_normal((Bn, H, S, dk)).astype(np.float32)  # plays dO; V below
    V = rng.standard_normal((Bn, H, S, dk)).astype(np.float32)
    scale = 0.125
    dq, dkk, ddo, dv = ctx.upload(Q), ctx.upload(Kx), ctx.upload(dPh), ctx.upload(V)
    P, dS = ctx.empty(Bn, H, S, S), ctx.empty(Bn, H, S, S)
    kw = dict(batch=(H, Bn), sA=(S * dk, H * S * dk), sB=(S * dk, H * S * dk), sC=(S * S, H * S * S), precision=prec)
    ctx.gemm(dq, dkk, P, S, S, dk, transB=True, alpha=scale, rowop=1, rowop_causal=causal, **kw)
    ctx.gemm(ddo, dv, dS, S, S, dk, transB=True, alpha=scale, rowop=2, rowop_aux=P, **kw)
    ops = orc.Ops(omp=True)
    Ph, dSh = P.numpy(), dS.numpy()
    for b in range(Bn):
        for h in range(H):
            s_ref = ops.matmul_fwd(w64(Q[b, h]), w64(Kx[b, h].T.copy())) * scale
            p_ref = ops.softmax_fwd(s_ref, S if causal else 0)
            assert rel(Ph[b, h], p_ref) <= 2 * tol  # softmax scales the error of the scores by their magnitude
            if causal:
                assert np.all(np.triu(Ph[b, h], 1) == 0.0)
            # backward on the GPU's own P (one product per tolerance)
            dp_ref = ops.matmul_fwd(w64(dPh[b, h]), w64(V[b, h].T.copy()))
            ds_ref = np.zeros((S, S))
            ops.softmax_bwd(w64(Ph[b, h]), dp_ref, ds_ref)
            assert rel(dSh[b, h], ds_ref * scale) <= 2 * tol


@pytest.mark.parametrize("kind,h,nstate", [(1, (0.9,), 1), (2, (0.9,), 1), (3, (0.9, 1e-8), 1), (4, (0.0, 1e-8), 1),
                                           (6, (0.9, 0.999, 1e-8, 0.01), 2), (7, (0.9, 0.999, 1e-8), 3)])
@pytest.mark.parametrize("n", [109386, 5])
def test_optimizer_family(ctx, orc, kind, h, nstate, n):
    """fml_optimizer_step against the oracle's restatement of lib/optimizers/{sgdmomentum,nag,rmsprop,adagrad,adamw,
    amsgrad}.dart over three steps with fresh gradients."""
    rng = np.random.default_rng(kind * 100 + n)
    w = rng.standard_normal(n).astype(np.float32)
    ops = orc.Ops()
    w_ref = w64(w)
    s_ref = [np.zeros(n) for _ in range(nstate)] + [None] * (3 - nstate)
    dw = ctx.upload(w)
    ds = [ctx.zeros(n) for _ in range(nstate)] + [None] * (3 - nstate)
    hh = tuple(h) + (0.0,) * (4 - len(h))
    for t in (1, 2, 3):
        g = rng.standard_normal(n).astype(np.float32)
        ops.optimizer_step(kind, w_ref, w64(g), s_ref[0], s_ref[1], s_ref[2], 1e-2, h, t)
        ctx.call("fml_optimizer_step", kind, dw, ctx.upload(g), ds[0], ds[1], ds[2], n, 1e-2, *hh, t)
    assert rel(dw.numpy(), w_ref) <= 1e-6
    for i in range(nstate):
        assert rel(ds[i].numpy(), s_ref[i]) <= 1e-6


def test_optimizer_family_rejects_bad_arguments(ctx):
    w, g = ctx.zeros(8), ctx.zeros(8)
    with pytest.raises(RuntimeError):
        ctx.call("fml_optimizer_step", 5, w, g, ctx.zeros(8), None, None, 8, 0.1, 0.9, 0.0, 0.0, 0.0, 1)   # unknown kind
    with pytest.raises(RuntimeError):
        ctx.call("fml_optimizer_step", 7, w, g, ctx.zeros(8), ctx.zeros(8), None, 8, 0.1, 0.9, 0.999, 1e-8, 0.0, 1)  # no s3


@pytest.mark.parametrize("kind,alpha", [(5, 0.01), (5, 0.3), (6, 1.0), (6, 0.5), (7, 0.0), (8, 0.0)])
def test_parameterised_activations(ctx, orc, kind, alpha):
    """fml_act2_fwd/bwd (LeakyReLU, ELU, Swish, Mish) against the oracle, including saturating inputs."""
    rng = np.random.default_rng(kind)
    x = np.concatenate([rng.standard_normal(70001) * 3, [0.0, -30.0, 30.0, 80.0, -80.0]]).astype(np.float32)
    dy = rng.standard_normal(x.size).astype(np.float32)
    ops = orc.Ops()
    y_ref = ops.act2_fwd(kind, alpha, w64(x))
    dx_ref = np.zeros(x.size)
    ops.act2_bwd(kind, alpha, w64(x), w64(dy), dx_ref)
    dxd, ddy, y, dx = ctx.upload(x), ctx.upload(dy), ctx.empty(x.size), ctx.empty(x.size)
    ctx.call("fml_act2_fwd", kind, alpha, dxd, y, x.size)
    ctx.call("fml_act2_bwd", kind, alpha, dxd, ddy, dx, x.size, 0)
    assert rel(y.numpy(), y_ref) <= 1e-6
    assert rel(dx.numpy(), dx_ref) <= 1e-6
    assert np.all(np.isfinite(y.numpy())) and np.all(np.isfinite(dx.numpy()))
    ctx.call("fml_act2_bwd", kind, alpha, dxd, ddy, dx, x.size, 1)   # accumulate
    assert rel(dx.numpy(), 2 * dx_ref) <= 1e-6


def test_bounded_wait_times_out_and_the_context_survives():
    """A device-side wait that nothing ever satisfies (the failure made by a barrier nobody signals, not by a fault):
    the kernel gives up after its limit, the host reads FML_ERR_TIMEOUT with the recorded code once, and the same
    context then runs a product correctly."""
    import ctypes
    from flutter_ml_b200 import _lib
    c = _lib.Context(precision=_lib.PREC_TF32)
    assert c.device_status() == 0
    c.check(c.lib.fml_selftest_wait_timeout(c.h, 2000))          # 2 ms
    code = ctypes.c_int32(0)
    assert c.lib.fml_device_status(c.h, ctypes.byref(code)) == -4   # FML_ERR_TIMEOUT
    assert code.value == 99 and b"bounded wait expired" in c.lib.fml_last_error(c.h)
    assert c.device_status() == 0                                 # reported once, then clear
    a = np.random.default_rng(0).standard_normal((256, 256)).astype(np.float32)
    A, B, C = c.upload(a), c.upload(a.T.copy()), c.empty(256, 256)
    c.gemm(A, B, C, 256, 256, 256)
    assert rel(C.numpy(), a.astype(np.float64) @ a.T.astype(np.float64)) <= TOL_TF32
    assert c.lib.fml_selftest_wait_timeout(c.h, 0) == -1          # limit out of range
    c.close()


@pytest.mark.parametrize("prec,tol", [(0, TOL_TF32), (1, 1e-5)])
def test_gemm_full_size_sampled_entries_and_exact_properties(prec, tol):
    """Config 2's largest square (8192^3), too large for the float64 oracle in full: 4096 randomly chosen output
    entries of C = A.B, dA = dC.B^T and dW = A^T.dC against exact float64 dot products of the same float32 operands,
    plus two size-independent properties: scaling an operand by a power of two scales the result bit-exactly, and
    (A.B)^T computed as B^T.A^T through the transposed-operand paths agrees with C."""
    from flutter_ml_b200 import _lib
    n = 8192
    c = _lib.Context(precision=prec)
    rng = np.random.default_rng(8192 + prec)
    A = (rng.standard_normal((n, n), dtype=np.float32) / np.float32(np.sqrt(n)))
    B = (rng.standard_normal((n, n), dtype=np.float32) / np.float32(np.sqrt(n)))
    dA_, dB_, C_, D_ = c.upload(A), c.upload(B), c.empty(n, n), c.empty(n, n)
    ii, jj = rng.integers(0, n, 4096), rng.integers(0, n, 4096)

    def sampled(got, left_rows, right_cols):     # got[i, j] vs sum_k left_rows[i, k] * right_cols[k, j]
        ref = np.einsum("sk,sk->s", left_rows.astype(np.float64), right_cols.astype(np.float64))
        return float(np.linalg.norm(got - ref) / np.linalg.norm(ref))

    c.gemm(dA_, dB_, C_, n, n, n)
    C = C_.numpy()
    assert sampled(C[ii, jj], A[ii, :], B[:, jj].T) <= tol
    # dA = dC . B^T with dC := C's operand role played by A (any matrix serves), dW = A^T . dC likewise
    c.gemm(dA_, dB_, D_, n, n, n, transB=True)
    assert sampled(D_.numpy()[ii, jj], A[ii, :], B[jj, :]) <= tol
    c.gemm(dA_, dB_, D_, n, n, n, transA=True)
    assert sampled(D_.numpy()[ii, jj], A[:, ii].T, B[:, jj].T) <= tol
    # (A.B)^T = B^T.A^T through both transposed-operand paths
    c.gemm(dB_, dA_, D_, n, n, n, transA=True, transB=True)
    Dt = D_.numpy()
    assert rel(Dt[jj, ii], C[ii, jj]) <= max(tol * 1e-2, 2e-6)
    # power-of-two scaling is exact in every rounding step
    c.call("fml_axpy", 3.0, dA_, dA_, n * n)          # A <- 4 A
    c.gemm(dA_, dB_, D_, n, n, n)
    assert np.array_equal(D_.numpy()[ii, jj], 4.0 * C[ii, jj])
    assert c.device_status() == 0
    c.close()


def test_out_of_range_ids_and_labels_are_reported_not_dereferenced(orc):
    """A token id outside the table or a label outside the logits (the reference would raise a RangeError,
    embeddingLayer.dart:53) is never used as an address: the kernels skip the access, fml_device_status returns
    FML_ERR_INVALID once with the kernel's code, memory next to the table is untouched and the context stays usable."""
    import ctypes
    from flutter_ml_b200 import _lib
    c = _lib.Context()
    V, d, n = 50, 8, 6
    rng = np.random.default_rng(3)
    # table sits in the middle of a larger buffer so that a stray write would be visible on either side
    guard = rng.standard_normal((3 * V, d)).astype(np.float32)
    buf = c.upload(guard)
    table = buf.view(V * d, (V, d))
    ids = np.array([3, V, 7, -1, 49, 1 << 30], dtype=np.int32)
    dids, out = c.upload(ids), c.empty(n, d)
    c.call("fml_embedding_fwd", table, dids, None, out, n, d, 0, V)
    code = ctypes.c_int32(0)
    assert c.lib.fml_device_status(c.h, ctypes.byref(code)) == -1 and code.value == 201
    assert b"token id" in c.lib.fml_last_error(c.h)
    assert c.device_status() == 0                                   # reported once
    got = out.numpy()
    ok = (ids >= 0) & (ids < V)
    assert np.array_equal(got[ok], guard[V:2 * V][ids[ok]]) and np.all(got[~ok] == 0)
    dout = c.upload(np.ones((n, d), np.float32))
    c.call("fml_embedding_bwd", dout, dids, table, n, d, V)         # adds into the table region only
    assert c.lib.fml_device_status(c.h, ctypes.byref(code)) == -1 and code.value == 202
    after = buf.numpy()
    assert np.array_equal(after[:V], guard[:V]) and np.array_equal(after[2 * V:], guard[2 * V:])
    expect = guard[V:2 * V].copy()
    for i in ids[ok]:
        expect[i] += 1
    assert np.array_equal(after[V:2 * V], expect)
    # labels: narrow rows (block-per-row kernel), wide rows (row-in-registers kernel), and the no-allocation entry point
    for cols, fn in ((10, "fml_softmax_xent"), (4096, "fml_softmax_xent"), (10, "fml_softmax_xent_static")):
        rows = 5
        z = rng.standard_normal((rows, cols)).astype(np.float32)
        labels = np.array([1, cols, 0, -3, cols - 1], dtype=np.int32)
        dz, loss = c.empty(rows, cols), c.zeros(1)
        c.call(fn, c.upload(z), c.upload(labels), dz, loss, rows, cols, 1.0 / rows, launches=2)
        assert c.lib.fml_device_status(c.h, ctypes.byref(code)) == -1 and code.value == 203, (cols, fn)
        good = (labels >= 0) & (labels < cols)
        ref_good = np.zeros((int(good.sum()), cols))
        ref_loss = orc.Ops().softmax_xent(w64(z[good]), np.ascontiguousarray(labels[good]), ref_good, 1.0 / rows)
        assert abs(loss.numpy()[0] - ref_loss) <= 1e-5 * abs(ref_loss), (cols, fn)   # bad rows add no loss
        assert rel(dz.numpy()[good], ref_good) <= 1e-5
        p = np.exp(w64(z[~good]) - w64(z[~good]).max(1, keepdims=True))
        assert rel(dz.numpy()[~good], p / p.sum(1, keepdims=True) / rows) <= 1e-5    # plain softmax, no one-hot term
    # the context still computes
    a = rng.standard_normal((64, 64)).astype(np.float32)
    C_ = c.empty(64, 64)
    c.gemm(c.upload(a), c.upload(a), C_, 64, 64, 64)
    assert rel(C_.numpy(), w64(a) @ w64(a)) <= TOL_TF32 and c.device_status() == 0
    c.close()


def test_one_host_thread_drives_several_contexts():
    """The reference's host is one isolate (lib/cuda/cudacaller.dart:25-60 runs on the caller's thread): one thread must be
    able to interleave calls on several contexts.  Two contexts on the same device always; one context per device on
    every visible GPU as well when there are several (each entry point makes its context's device current, and the
    kernels' shared-memory opt-in is made once per device)."""
    import ctypes
    from flutter_ml_b200 import _lib
    n_dev = ctypes.c_int32(0)
    assert _lib.load().fml_device_count(ctypes.byref(n_dev)) == 0
    devices = [0, 0] + list(range(1, min(n_dev.value, 4)))
    ctxs = [_lib.Context(device=dv, precision=_lib.PREC_TF32) for dv in devices]
    rng = np.random.default_rng(17)
    M, N, K = 384, 320, 256                                         # tensor-core path: needs the shared-memory opt-in
    jobs = []
    for i, c in enumerate(ctxs):                                    # enqueue on every context before reading any result
        a, b = rng.standard_normal((M, K)).astype(np.float32), rng.standard_normal((K, N)).astype(np.float32)
        A, B, C_ = c.upload(a), c.upload(b), c.empty(M, N)
        jobs.append((c, a, b, A, B, C_))
    for c, a, b, A, B, C_ in jobs:
        c.gemm(A, B, C_, M, N, K, act="gelu", bias=None)
        assert c.gemm_last_path() == 1
    for c, a, b, A, B, C_ in reversed(jobs):
        z = w64(a) @ w64(b)
        from math import sqrt
        from scipy.special import erf
        assert rel(C_.numpy(), 0.5 * z * (1 + erf(z / sqrt(2)))) <= TOL_TF32
        assert c.device_status() == 0
    for c in ctxs:
        c.close()


def test_communicator_creation_times_out_when_the_peer_never_joins():
    """Failure made on the host, no kernel involved: rank 0 of a world of two whose peer never calls in.  The
    non-blocking communicator creation is polled against the limit, aborted when it passes, and reported as
    FML_ERR_TIMEOUT; the context then still computes and can join a new (single-rank) world."""
    import ctypes
    import os
    import time
    from flutter_ml_b200 import _lib
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    c = _lib.Context()
    uid = ctypes.create_string_buffer(128)
    assert c.lib.fml_dp_unique_id(uid) == 0
    assert c.lib.fml_dp_set_timeout(c.h, 0) == -1
    c.check(c.lib.fml_dp_set_timeout(c.h, 1500))
    t0 = time.time()
    rc = c.lib.fml_dp_init(c.h, uid.raw, 0, 2)
    waited = time.time() - t0
    assert rc == -4, (rc, c.lib.fml_last_error(c.h))
    assert b"a peer did not arrive" in c.lib.fml_last_error(c.h)
    assert 1.0 <= waited <= 20.0, waited
    assert c.lib.fml_dp_allreduce_sum(c.h, None, 0) == 0             # back to a world of one: nothing to exchange
    a = np.random.default_rng(1).standard_normal((128, 128)).astype(np.float32)
    C_ = c.empty(128, 128)
    c.gemm(c.upload(a), c.upload(a), C_, 128, 128, 128)
    assert rel(C_.numpy(), w64(a) @ w64(a)) <= TOL_TF32 and c.device_status() == 0
    c.check(c.lib.fml_dp_init(c.h, bytes(128), 0, 1))
    c.close()


@pytest.mark.parametrize("M,N,K,tA,tB", [(384, 320, 256, 0, 0), (2048, 2048, 512, 0, 0), (2048, 2048, 512, 0, 1), (2048, 2048, 512, 1, 0),
                                         (300, 200, 100, 1, 1), (1024, 1024, 8192, 1, 0)])
def test_tf32_product_is_the_exact_product_of_truncated_operands(ctx, M, N, K, tA, tB):
    """Where the TF32 error comes from: the tensor core drops the low 13 mantissa bits of every fp32 operand and then
    multiplies and accumulates (in fp32) without further loss.  A float64 product of operands cut to 19 bits on the
    host must therefore reproduce the device result to fp32 accumulation accuracy, in every tile mode and operand
    layout; the distance of both from the exact product is the operand truncation alone (about 7.7e-4 on generic
    data, of which 7.0e-4 is a bias toward zero: 3.5e-4 per operand)."""
    rng = np.random.default_rng(M + N + K + tA + 2 * tB)
    A = rng.standard_normal((K, M) if tA else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if tB else (K, N)).astype(np.float32)
    dC = ctx.empty(M, N)
    ctx.gemm(ctx.upload(A), ctx.upload(B), dC, M, N, K, transA=bool(tA), transB=bool(tB), precision=0)
    assert ctx.gemm_last_path() == 1

    def cut(x):
        return (np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32).astype(np.float64)
    opA, opB = (A.T if tA else A), (B.T if tB else B)
    got = dC.numpy()
    # fp32 accumulation inside the tensor core: its error grows with the length of the chain (about 1.5e-9 per term)
    assert rel(got, cut(opA) @ cut(opB)) <= max(3e-6, 3e-9 * K), rel(got, cut(opA) @ cut(opB))
    exact = w64(opA) @ w64(opB)
    assert 4e-4 <= rel(got, exact) <= TOL_TF32
    shrink = float(np.sum(got * exact) / np.sum(exact * exact)) - 1.0          # least-squares scale of got against exact
    assert -9e-4 <= shrink <= -5e-4, shrink


@pytest.mark.parametrize("T,B,I,H", [(6, 128, 16, 256), (5, 70, 8, 512), (3, 3, 4, 128), (1, 9, 4, 128), (9, 33, 12, 384), (40, 128, 8, 512)])
def test_lstm_fused_step_backward_recurrence(orc, T, B, I, H):
    """The default backward recurrence in TF32 mode at batch <= 128 and H a multiple of 128 up to 512: one launch per step
    that forms the gate derivatives, multiplies by Wh and sums the sixteen slices of the contraction with bulk reduce-add
    copies, the steps chained by programmatic dependent launch.  Against the oracle's BPTT (lstmLayer.dart:112-150 walked
    backwards) for dW and db, and against the gate kernel + K-split product per step (FML_LSTM_BWD_FUSED=0) for the dpre of
    every step: the same TF32 products of the same operands, summed in another order."""
    import ctypes
    import os
    from flutter_ml_b200 import _lib
    c = _lib.Context(precision=_lib.PREC_TF32)
    rng = np.random.default_rng(100 * T + H + B + 1)
    a = 1 / np.sqrt(H)
    W = rng.uniform(-a, a, (4, H, H + I)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (4, H)).astype(np.float32)
    x = rng.standard_normal((B, T, I)).astype(np.float32)
    target = rng.standard_normal((B, H)).astype(np.float32)
    h_ref, loss_ref, dW_ref, db_ref = orc.Ops(omp=True).lstm_fwd_bwd(w64(W), w64(b), w64(x), w64(target))
    d = _lib.LstmDesc()
    d.T, d.B, d.I, d.H = T, B, I, H
    bufs = dict(W=c.upload(W), b=c.upload(b), x=c.upload(np.ascontiguousarray(x.transpose(1, 0, 2))),
                gates=c.empty(T, B, 4 * H), cells=c.empty(T + 1, B, H), hs=c.empty(T + 1, B, H), xproj=c.empty(T * B, 4 * H))
    for k, v in bufs.items():
        setattr(d, k, v.ptr)
    c.check(c.lib.fml_lstm_fwd(c.h, ctypes.byref(d)))
    h_last = bufs["hs"].view(T * B * H, (B, H))
    dh, loss = c.empty(B, H), c.zeros(1)
    c.call("fml_mse", h_last, c.upload(target), dh, loss, B * H, float(B))
    scratch = c.empty(T * B * 4 * H + 2 * B * H)
    runs = {}
    try:
        for fused in ("1", "0"):
            os.environ["FML_LSTM_BWD_FUSED"] = fused
            dW_, db_, dx_ = c.zeros(4 * H, H + I), c.zeros(4 * H), c.empty(T * B, I)
            c.check(c.lib.fml_lstm_bwd(c.h, ctypes.byref(d), dh.ptr, dW_.ptr, db_.ptr, dx_.ptr, scratch.ptr))
            assert c.device_status() == 0
            runs[fused] = (scratch.numpy()[:T * B * 4 * H].copy(), dW_.numpy().copy(), db_.numpy().copy(), dx_.numpy().copy())
    finally:
        os.environ.pop("FML_LSTM_BWD_FUSED", None)
    dpre, dW_g, db_g, dx_g = runs["1"]
    assert rel(dW_g.reshape(4, H, H + I), dW_ref) <= 2 * TOL_TF32
    assert rel(db_g.reshape(4, H), db_ref) <= 2 * TOL_TF32
    # step by step against the two-launch path (the last step first: it involves no product at all)
    per = B * 4 * H
    for t in range(T - 1, -1, -1):
        r_t = rel(dpre[t * per:(t + 1) * per], runs["0"][0][t * per:(t + 1) * per])
        # equal up to the order of the fp32 sums at the last step; each further step rounds the slightly different dpre
        # to TF32 again, so the two chains drift apart by a few 1e-6 per step (measured 2.1e-5 after eight)
        assert r_t <= 1e-5 * (T - t), (t, r_t)
    assert rel(dx_g, runs["0"][3]) <= 1e-5 * T
    c.close()


@pytest.mark.parametrize("T,B,I,H", [(6, 128, 16, 256), (5, 70, 8, 512), (3, 3, 4, 128), (1, 9, 4, 128), (9, 33, 12, 384)])
def test_lstm_single_kernel_backward_recurrence(orc, T, B, I, H):
    """The opt-in cooperative backward kernel (TF32 mode, batch <= 128, H a multiple of 128 up to 512: the contraction split
    over a cluster of sixteen CTAs and summed in a fixed order through distributed shared memory) against the oracle's BPTT (lstmLayer.dart:112-150 walked backwards): dW and db; and run twice to show
    that the recurrence is bit-for-bit reproducible, which the K split with atomics it replaces was not."""
    import ctypes
    import os
    from flutter_ml_b200 import _lib
    os.environ["FML_LSTM_BWD_SINGLE_KERNEL"] = "1"      # opt-in: the default is two launches per step (faster, not reproducible)
    c = _lib.Context(precision=_lib.PREC_TF32)
    rng = np.random.default_rng(100 * T + H + B)
    a = 1 / np.sqrt(H)
    W = rng.uniform(-a, a, (4, H, H + I)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (4, H)).astype(np.float32)
    x = rng.standard_normal((B, T, I)).astype(np.float32)
    target = rng.standard_normal((B, H)).astype(np.float32)
    h_ref, loss_ref, dW_ref, db_ref = orc.Ops(omp=True).lstm_fwd_bwd(w64(W), w64(b), w64(x), w64(target))
    d = _lib.LstmDesc()
    d.T, d.B, d.I, d.H = T, B, I, H
    bufs = dict(W=c.upload(W), b=c.upload(b), x=c.upload(np.ascontiguousarray(x.transpose(1, 0, 2))),
                gates=c.empty(T, B, 4 * H), cells=c.empty(T + 1, B, H), hs=c.empty(T + 1, B, H), xproj=c.empty(T * B, 4 * H))
    for k, v in bufs.items():
        setattr(d, k, v.ptr)
    c.check(c.lib.fml_lstm_fwd(c.h, ctypes.byref(d)))
    h_last = bufs["hs"].view(T * B * H, (B, H))
    dh, loss = c.empty(B, H), c.zeros(1)
    c.call("fml_mse", h_last, c.upload(target), dh, loss, B * H, float(B))
    scratch = c.empty(T * B * 4 * H + 2 * B * H)
    runs = []
    for _ in range(2):
        dW_, db_, dx_ = c.zeros(4 * H, H + I), c.zeros(4 * H), c.empty(T * B, I)
        c.check(c.lib.fml_lstm_bwd(c.h, ctypes.byref(d), dh.ptr, dW_.ptr, db_.ptr, dx_.ptr, scratch.ptr))
        assert c.device_status() == 0
        runs.append((scratch.numpy()[:T * B * 4 * H].copy(), dx_.numpy()))
    assert rel(h_last.numpy(), h_ref) <= TOL_TF32
    assert rel(dW_.numpy().reshape(4, H, H + I), dW_ref) <= 2 * TOL_TF32
    assert rel(db_.numpy().reshape(4, H), db_ref) <= 2 * TOL_TF32
    assert np.array_equal(runs[0][0], runs[1][0])      # dpre of every step, i.e. the whole dh chain, bit for bit
    os.environ.pop("FML_LSTM_BWD_SINGLE_KERNEL")
    c.close()
