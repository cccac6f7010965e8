"""Model-level parity: the reference-shaped layers on the GPU against the oracle's tape."""
import numpy as np
import pytest

from tests.gpu_util import rel

pytestmark = pytest.mark.gpu
w64 = lambda x: np.ascontiguousarray(x, dtype=np.float64)  # noqa: E731

# Whole-model tolerances (relative Frobenius error vs the float64 oracle): (outputs, gradients).
#  - 3xTF32: 1e-5 for both, the tolerance stated for one product.  Measured on these three models: logits / outputs
#    5e-7 .. 2.3e-6, gradients 7e-7 .. 6.8e-6 (the deepest chain, the language model's embedding gradient); every test
#    prints its figures.  This mode pins the LOGIC of every layer and of the tape.
#  - TF32: a single product is within 1e-3 (5.5e-4 measured, test_gpu_kernels.py); outputs of a chain of
#    products are held to 2e-3.  Gradients of these three models pass through ReLU gates
#    (tensor.dart:1030), which are discontinuous: a pre-activation within ~5e-4 of zero can land on the
#    other side of the gate than in float64, and a fraction f of flipped gates gives a relative gradient
#    error of about sqrt(f) (f ~ 5e-4 -> ~2e-2) for ANY TF32 product, however exact the kernel is.  The
#    gradient bound in TF32 mode is therefore 5e-2; per-kernel gradient parity at 1e-3 is asserted in
#    test_gpu_kernels.py on identical gate inputs.
TOLS = {0: (2e-3, 5e-2), 1: (1e-5, 1e-5)}


@pytest.mark.parametrize("prec", [0, 1])
def test_mlp_training_step_config1(orc, prec):
    """Config 1 at full size: 784-128-64-10, batch 64, seed 0, one SGD step."""
    from flutter_ml_b200 import _lib, models, synth
    ctx = _lib.Context(precision=prec)
    params = models.init_mlp(0)
    X = synth.uniform(0, 0, (64, 784))
    labels = synth.integers(0, 1, (64,), 10)
    ref = orc.mlp_step(w64(X), labels, [w64(p) for p in params], lr=0.01, omp=True)
    mlp = models.MLP(ctx, params, lr=0.01)
    loss, logits, grads = mlp.train_step(ctx.upload(X), ctx.upload(labels), keep=True)
    t_out, t_grad = TOLS[prec]
    lg = logits.numpy()
    flat_ref_ = np.concatenate([np.pad(g.ravel(), (0, (-g.size) % 4)) for g in ref["grads"]])
    print(f"PARITY config1 prec{prec}: logits {rel(lg, ref['logits']):.2e} gradients {rel(grads, flat_ref_):.2e}")
    assert rel(lg, ref["logits"]) <= t_out
    assert np.array_equal(lg.argmax(1), ref["logits"].argmax(1))      # argmax-identical logits
    assert abs(loss.numpy()[0] - ref["loss"]) <= t_out * abs(ref["loss"])
    flat_ref = np.concatenate([np.pad(g.ravel(), (0, (-g.size) % 4)) for g in ref["grads"]])
    assert rel(grads, flat_ref) <= t_grad
    new = mlp.arena.values.numpy()
    flat_new = np.concatenate([np.pad(p.ravel(), (0, (-p.size) % 4)) for p in ref["params"]])
    # the update is w - lr*g: the gradient tolerance above, scaled by lr*|g|/|w|
    assert rel(new, flat_new) <= (1e-4 if prec == 0 else 1e-5)
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("causal", [True, False])
def test_encoder_block_config3_scaled(orc, prec, causal):
    """Config 3's block (post-LN, ReLU FFN, causal attention) at d=128, 4 heads, dff 256, seq 64, 3 sequences."""
    from flutter_ml_b200 import _lib, models, synth
    ctx = _lib.Context(precision=prec)
    d, heads, dff, S, B = 128, 4, 256, 64, 3
    p = models.init_block(2, d, heads, dff, std=0.08)
    x, tgt = synth.normal(2, 500, (B, S, d)), synth.normal(2, 501, (B, S, d))
    p64 = {k: (w64(v) if k != "heads" else [tuple(w64(w) for w in h) for h in v]) for k, v in p.items()}
    ref = orc.encoder_block_fwd_bwd(w64(x), p64, w64(tgt), causal, omp=True)
    y, loss, dx, grads = models.encoder_block_fwd_bwd(ctx, x, p, tgt, heads, causal)
    t_out, t_grad = TOLS[prec]
    print(f"PARITY block-scaled prec{prec} causal {causal}: y {rel(y, ref['y']):.2e} dx {rel(dx, ref['dx']):.2e} "
          f"worst weight gradient {max(rel(g, r) for g, r in zip(grads, ref['grads'])):.2e}")
    assert rel(y, ref["y"]) <= t_out
    assert abs(loss - ref["loss"]) <= t_out * abs(ref["loss"])
    assert rel(dx, ref["dx"]) <= t_grad
    for g, r in zip(grads, ref["grads"]):
        assert rel(g, r) <= t_grad
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_transformer_lm_step_config5_scaled(orc, prec):
    """Config 5 scaled down (2 layers, d 128, 4 heads, dff 256, seq 32, vocab 1000, batch 4): loss, logits
    argmax, every gradient, and the Adam update."""
    from flutter_ml_b200 import _lib, models, synth
    ctx = _lib.Context(precision=prec)
    V, d, heads, dff, L, S, B = 1000, 128, 4, 256, 2, 32, 4
    params = models.init_lm(4, V, d, heads, dff, L, std=0.05)
    ids, labels = synth.integers(4, 100, (B, S), V), synth.integers(4, 101, (B, S), V)
    conv = lambda b: {k: (w64(v) if k != "heads" else [tuple(w64(w) for w in h) for h in v]) for k, v in b.items()}  # noqa: E731
    p64 = {"emb": w64(params["emb"]), "blocks": [conv(b) for b in params["blocks"]], "Whead": w64(params["Whead"]),
           "bhead": w64(params["bhead"])}
    ref = orc.lm_forward_backward(ids, labels, p64, B * S, True, omp=True)
    lm = models.TransformerLM(ctx, params, S, heads, lr=1e-3)
    loss, logits = lm.forward_backward(ctx.upload(ids.reshape(-1)), ctx.upload(labels.reshape(-1)), B * S, keep_logits=True)
    t_out, t_grad = TOLS[prec]
    lg = logits.numpy().reshape(B, S, V)
    assert rel(lg, ref["logits"]) <= t_out
    # Argmax: identical on every row whose float64 top-2 margin exceeds twice the largest logit error measured here (such a
    # row cannot flip); the rows below that margin are near-ties among 1000 random logits and are counted, not asserted.
    r64 = ref["logits"].reshape(-1, V)
    top2 = np.sort(r64, axis=1)[:, -2:]
    margin = top2[:, 1] - top2[:, 0]
    max_err = float(np.max(np.abs(lg.reshape(-1, V) - r64)))
    same = lg.reshape(-1, V).argmax(1) == r64.argmax(1)
    safe = margin > 2 * max_err
    print(f"PARITY lm-head argmax prec{prec}: rows {same.size}, max |logit error| {max_err:.2e}, top-2 margin min {margin.min():.2e} "
          f"median {np.median(margin):.2e}, rows with margin <= 2 max error: {int((~safe).sum())}, of which flipped: {int((~same & ~safe).sum())}")
    assert same[safe].all()
    if prec == 1:
        assert same.all()
    assert abs(loss.numpy()[0] - ref["loss"]) <= t_out * abs(ref["loss"])
    g_errs = [rel(g, r) for g, r in zip(lm.grads_in_reference_order(), ref["grads"])]
    print(f"PARITY lm-scaled prec{prec}: logits {rel(lg, ref['logits']):.2e} worst gradient {max(g_errs):.2e} median {np.median(g_errs):.2e}")
    for e in g_errs:
        assert e <= t_grad
    # Adam step on the whole arena equals the oracle's per-tensor update
    ops = orc.Ops()
    g_flat = lm.arena.grads.numpy().astype(np.float64)
    w_flat = lm.arena.values.numpy().astype(np.float64)
    m, v = np.zeros_like(w_flat), np.zeros_like(w_flat)
    ops.adam_step(w_flat, g_flat, m, v, 1e-3, 1)
    lm.optimizer.step()
    assert rel(lm.arena.values.numpy(), w_flat) <= 1e-6
    assert ctx.device_status() == 0
    ctx.close()


def test_snetwork_fit_xor():
    """The reference's XOR demo (lib/nets/snet.dart:159-227): per-sample fit with mse lowers the loss."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.layers import DenseLayerMatrix
    from flutter_ml_b200.optimizers import SGD
    from flutter_ml_b200.snet import SNetwork
    from flutter_ml_b200.tensor import Tensor, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    set_default_context(ctx)
    net = SNetwork([DenseLayerMatrix(8, "tanh", seed=5), DenseLayerMatrix(1, "sigmoid", seed=6)])
    xs = [Tensor(np.array([[a, b]], dtype=np.float32), ctx) for a in (0, 1) for b in (0, 1)]
    ys = [Tensor(np.array([[float(a ^ b)]], dtype=np.float32), ctx) for a in (0, 1) for b in (0, 1)]
    net.predict(xs[0])
    net.compile(SGD(net.parameters, 0.5))
    hist = net.fit(xs, ys, epochs=300)
    assert hist[-1] < 0.5 * hist[0]
    assert net.evaluate(xs, ys) >= 0.75
    ctx.close()


def test_cudacaller_matmult_signature():
    """CudaCaller.matmult(A, B, m, k, n) -> flat list of doubles (lib/cuda/cudacaller.dart:25-60)."""
    from flutter_ml_b200.cuda import CudaCaller
    m, k, n = 8, 16, 4
    out = CudaCaller.matmult([1.0] * (m * k), [1.0] * (k * n), m, k, n)
    assert isinstance(out, list) and len(out) == m * n and all(v == float(k) for v in out)


def test_pipelined_host_step_equals_serial():
    """ops.DenseFwdBwdHost: the overlapped form (copy lanes + two buffer sets) returns what the serial form does."""
    from flutter_ml_b200 import _lib, ops, synth
    ctx = _lib.Context()
    M, N, K = 384, 320, 256
    host = ops.DenseFwdBwdHost(ctx, M, N, K, act="gelu")
    for i, k in enumerate(("A", "B", "bias", "dC")):
        host.h_in[k][...] = synth.normal(1, i, host.h_in[k].shape, 1 / np.sqrt(K))
    ref = {k: v.copy() for k, v in host().items()}
    for v in host.h_out.values():
        v[...] = 0
    out = host.pipelined(5)
    for k in ref:
        # identical kernels on identical inputs; only sums formed with atomics (dbias, split-K products)
        # may differ in the last bit between runs
        assert np.allclose(out[k], ref[k], rtol=1e-5, atol=1e-6), k
    assert ctx.device_status() == 0
    ctx.close()


def test_optional_epilogue_fusions_give_the_same_gradients(orc):
    """tensor.FUSE_DACT_INTO_DX / FUSE_SOFTMAX_BACKWARD (off by default because they measured slower) against the
    default path, on the encoder block."""
    from flutter_ml_b200 import _lib, models, synth
    from flutter_ml_b200 import tensor as T
    ctx = _lib.Context(precision=_lib.PREC_3XTF32)
    d, heads, dff, S, B = 128, 4, 256, 64, 2
    p = models.init_block(2, d, heads, dff, std=0.08)
    x, tgt = synth.normal(2, 500, (B, S, d)), synth.normal(2, 501, (B, S, d))
    base = models.encoder_block_fwd_bwd(ctx, x, p, tgt, heads, True)
    T.FUSE_DACT_INTO_DX = T.FUSE_SOFTMAX_BACKWARD = True
    try:
        fused = models.encoder_block_fwd_bwd(ctx, x, p, tgt, heads, True)
    finally:
        T.FUSE_DACT_INTO_DX = T.FUSE_SOFTMAX_BACKWARD = False
    assert rel(fused[2], base[2]) <= 2e-5
    for g, r in zip(fused[3], base[3]):
        assert rel(g, r) <= 2e-5
    ctx.close()


def test_mlp_step_recorded_as_cuda_graph_matches_eager_steps():
    """fml_graph_*: N replays of the recorded MLP training step leave the parameters where N eager steps do."""
    from flutter_ml_b200 import _lib, models, synth
    ctx = _lib.Context()
    params = models.init_mlp(0)
    X, labels = ctx.upload(synth.uniform(0, 0, (64, 784))), ctx.upload(synth.integers(0, 1, (64,), 10))
    eager, graph = models.MLP(ctx, params, lr=0.01), models.MLP(ctx, params, lr=0.01)
    graph.record_step(X, labels)            # runs one eager step and one recorded (not executed) step
    for _ in range(4):
        graph.replay_step()
    for _ in range(5):
        loss, _, _ = eager.train_step(X, labels)
    a, b = graph.arena.values.numpy(), eager.arena.values.numpy()
    assert rel(a, b) <= 1e-6                # split-K / bias sums use atomics: last-bit differences only
    assert abs(graph.loss.numpy()[0] - loss.numpy()[0]) <= 1e-5 * abs(loss.numpy()[0])
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("act", ["leaky_relu", "elu", "swish", "mish"])
@pytest.mark.parametrize("opt_name", ["SGDMomentum", "NAG", "RMSprop", "Adagrad", "AdamW", "AMSGrad"])
def test_dense_net_with_other_activations_and_optimizers(orc, act, opt_name):
    """Two dense layers with one of the remaining activation functions, trained two steps with one of the remaining
    optimizers (flat parameter arena): parameters after the steps against the same steps in the oracle."""
    from flutter_ml_b200 import _lib, optimizers
    from flutter_ml_b200.layers import DenseLayerMatrix
    from flutter_ml_b200.tensor import Tensor, mseMatrix, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    set_default_context(ctx)
    rng = np.random.default_rng(11)
    Bn, din, dh, dout = 32, 24, 40, 8
    X, Y = rng.standard_normal((Bn, din)).astype(np.float32), rng.standard_normal((Bn, dout)).astype(np.float32)
    l1, l2 = DenseLayerMatrix(dh, act, seed=1), DenseLayerMatrix(dout, None, seed=2)
    x = Tensor(X, ctx)
    l2(l1(x))
    params = l1.parameters + l2.parameters
    ref = [p.numpy(np.float64).copy() for p in params]
    arena = optimizers.ParameterArena(ctx, params)
    kind, h, nstate = {"SGDMomentum": (1, (0.9,), 1), "NAG": (2, (0.9,), 1), "RMSprop": (3, (0.99, 1e-8), 1),   # the reference's default beta (rmsprop.dart:28)
                      
                       "Adagrad": (4, (0.0, 1e-8), 1), "AdamW": (6, (0.9, 0.999, 1e-8, 0.01), 2),
                       "AMSGrad": (7, (0.9, 0.999, 1e-8), 3)}[opt_name]
    opt = getattr(optimizers, opt_name)(params, 0.01, arena=arena)
    ops = orc.Ops()
    code, alpha = {"leaky_relu": (5, 0.01), "elu": (6, 1.0), "swish": (7, 0.0), "mish": (8, 0.0)}[act]
    state = [[np.zeros(r.size) for _ in range(nstate)] + [None] * (3 - nstate) for r in ref]
    X64, Y64 = X.astype(np.float64), Y.astype(np.float64)
    for t in (1, 2):
        opt.zeroGrad()
        loss = mseMatrix(l2(l1(Tensor(X, ctx))), Tensor(Y, ctx))
        loss.backward()
        opt.step()
        W1, b1, W2, b2 = ref
        z = X64 @ W1 + b1
        a = ops.act2_fwd(code, alpha, np.ascontiguousarray(z))
        out = a @ W2 + b2
        dout_ = 2.0 * (out - Y64) / out.size
        gW2, gb2 = a.T @ dout_, dout_.sum(0)
        da = np.ascontiguousarray(dout_ @ W2.T)
        dz = np.zeros_like(z)
        ops.act2_bwd(code, alpha, np.ascontiguousarray(z), da, dz)
        gW1, gb1 = X64.T @ dz, dz.sum(0)
        if t == 1:
            assert abs(float(loss.numpy().ravel()[0]) - float(((out - Y64) ** 2).mean())) <= 1e-5 * float(((out - Y64) ** 2).mean())
        for r, g, s in zip(ref, (gW1, gb1, gW2, gb2), state):
            rf, gf = r.reshape(-1), np.ascontiguousarray(g.reshape(-1))
            ops.optimizer_step(kind, rf, gf, s[0], s[1], s[2], 0.01, h, t)
    for p, r in zip(params, ref):
        assert rel(p.numpy(), r) <= 2e-5
    ctx.close()


@pytest.mark.parametrize("padding", ["valid", "same"])
def test_conv2d_layer_batched(orc, padding):
    """Conv2DLayer (lib/layertypes/conv2d.dart:60-75) over a batch of images in one launch: every feature map and
    every gradient against per-image, per-kernel conv2d + addScalarToMatrix on the oracle's tape."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.layers import Conv2DLayer
    from flutter_ml_b200.tensor import Tensor, mseMatrix, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    set_default_context(ctx)
    rng = np.random.default_rng(4)
    n_img, H, W, n_k, k = 5, 20, 33, 6, 3
    X = rng.standard_normal((n_img, H, W)).astype(np.float32)
    Kn = (rng.standard_normal((n_k, k * k)) * 0.5).astype(np.float32)
    Bv = rng.standard_normal(n_k).astype(np.float32)
    layer = Conv2DLayer(n_k, k, padding, kernels=Kn, biases=Bv)
    x = Tensor(X, ctx)
    out = layer(x)
    target = np.zeros(out.shape, np.float32)
    loss = mseMatrix(out, Tensor(target, ctx))
    loss.backward()
    E = orc.Engine()
    ok = [orc.T(Kn[c].reshape(k, k).astype(np.float64)) for c in range(n_k)]
    ob = [orc.T(np.float64(Bv[c])) for c in range(n_k)]
    ox = [orc.T(X[b].astype(np.float64)) for b in range(n_img)]
    maps = [[E.addScalarToMatrix(E.conv2d(ox[b], ok[c], padding), ob[c]) for c in range(n_k)] for b in range(n_img)]
    ref = np.stack([np.stack([m.value for m in row]) for row in maps])
    assert rel(out.numpy(), ref) <= 2e-6
    # d(mean over all elements of out^2): seed every map with its slice of the gradient and run its closures
    for b in range(n_img):
        for c in range(n_k):
            m = maps[b][c]
            m.grad = 2.0 * m.value / ref.size
            m.backward_fn()                 # addScalarToMatrix
            m.inputs[0].backward_fn()       # conv2d
    assert rel(x.grad_numpy(), np.stack([t.grad for t in ox])) <= 1e-5
    assert rel(layer.kernels.grad_numpy(), np.stack([t.grad.ravel() for t in ok])) <= 1e-5
    assert rel(layer.biases.grad_numpy(), np.array([float(t.grad) for t in ob])) <= 1e-5
    ctx.close()


@pytest.mark.parametrize("B", [1, 6])
def test_lstm_layer_mirror(orc, B):
    """layers.LSTMLayer (lib/layertypes/lstmLayer.dart:37-151) on one sequence [T x I] and on a time-major batch:
    last hidden state and the eight parameter gradients (handed out in the reference's order W_f, b_f, W_i, ...)
    against the oracle's step-by-step recurrence and BPTT."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.layers import LSTMLayer
    from flutter_ml_b200.tensor import Tensor
    ctx = _lib.Context(precision=_lib.PREC_3XTF32)
    Tn, I, H = 9, 5, 16
    rng = np.random.default_rng(23 + B)
    a = 1 / np.sqrt(H + I)
    W = rng.uniform(-a, a, (4, H, H + I)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (4, H)).astype(np.float32)
    x = rng.standard_normal((B, Tn, I)).astype(np.float32)
    target = rng.standard_normal((B, H)).astype(np.float32)
    h_ref, loss_ref, dW_ref, db_ref = orc.Ops(omp=True).lstm_fwd_bwd(w64(W), w64(b), w64(x), w64(target))
    layer = LSTMLayer(H, weights=W.reshape(4 * H, H + I), bias=b.reshape(4 * H))
    xin = x[0] if B == 1 else np.ascontiguousarray(x.transpose(1, 0, 2))
    out = layer(Tensor(xin, ctx))
    assert out.shape == (B, H) and len(layer.parameters) == 8
    loss = T.mseMatrix(out, Tensor(target, ctx))          # mean over B*H = (sum over sequences of mse) / B
    loss.backward()
    assert rel(out.numpy(), h_ref) <= 1e-5
    assert abs(loss.numpy()[0] * B - loss_ref) <= 1e-5 * abs(loss_ref)
    for g in range(4):
        Wg, bg = layer.parameters[2 * g], layer.parameters[2 * g + 1]
        assert np.array_equal(Wg.numpy(), W[g]) and np.array_equal(bg.numpy(), b[g])
        assert rel(Wg.grad_numpy() * B, dW_ref[g]) <= 2e-5
        assert rel(bg.grad_numpy() * B, db_ref[g]) <= 2e-5
    assert ctx.device_status() == 0
    ctx.close()


def test_snetwork_with_lstm_layer_learns_a_sequence_task():
    """SNetwork([LSTMLayer, DenseLayerMatrix]) trained per sample with fit(), the shape of the reference's
    sequence demos (lib/layertypes/lstmLayer.dart:153-260): next value of a sine wave from the last 8."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.layers import DenseLayerMatrix, LSTMLayer
    from flutter_ml_b200.optimizers import Adam
    from flutter_ml_b200.snet import SNetwork
    from flutter_ml_b200.tensor import Tensor, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    set_default_context(ctx)
    t = np.arange(0, 40) * 0.35
    wave = np.sin(t).astype(np.float32)
    xs = [Tensor(wave[i:i + 8].reshape(8, 1), ctx) for i in range(24)]
    ys = [Tensor(wave[i + 8].reshape(1, 1), ctx) for i in range(24)]
    net = SNetwork([LSTMLayer(12, seed=3), DenseLayerMatrix(1, None, seed=4)])
    net.predict(xs[0])
    assert len(net.parameters) == 10
    net.compile(Adam(net.parameters, 0.02))
    hist = net.fit(xs, ys, epochs=12)
    assert hist[-1] < 0.25 * hist[0]
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("act", [None, "tanh", "relu"])
def test_dense_layer_vector_form(orc, act):
    """layers.DenseLayer (lib/layertypes/denseLayer.dart:15-64): act(W.x + b) with W [out x in], stacked twice so
    the input gradient path through the first layer is exercised; against matVecMul + addVector on the oracle."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.layers import DenseLayer
    from flutter_ml_b200.tensor import Tensor
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    rng = np.random.default_rng(3)
    n_in, n_mid, n_out = 12, 9, 4
    W1, b1 = rng.standard_normal((n_mid, n_in)).astype(np.float32) * 0.4, rng.standard_normal(n_mid).astype(np.float32) * 0.1
    W2, b2 = rng.standard_normal((n_out, n_mid)).astype(np.float32) * 0.4, rng.standard_normal(n_out).astype(np.float32) * 0.1
    x, target = rng.standard_normal(n_in).astype(np.float32), rng.standard_normal(n_out).astype(np.float32)
    l1, l2 = DenseLayer(n_mid, act, weights=W1, bias=b1), DenseLayer(n_out, None, weights=W2, bias=b2)
    out = l2(l1(Tensor(x, ctx)))
    assert out.shape == (1, n_out) and l1.weights.shape == (n_mid, n_in)
    loss = T.mseMatrix(out, Tensor(target.reshape(1, -1), ctx))
    loss.backward()
    E = orc.Engine()
    oW1, ob1, oW2, ob2 = (orc.T(w64(a)) for a in (W1, b1, W2, b2))
    h = E.addMatrix(E.matVecMul(oW1, orc.T(w64(x))), ob1)
    if act:
        h = {"tanh": E.tanhMatrix, "relu": E.reluMatrix}[act](h)
    o = E.addMatrix(E.matVecMul(oW2, h), ob2)
    ol = E.mseMatrix(o, orc.T(w64(target)))
    ol.backward()
    assert rel(out.numpy().ravel(), o.value) <= 1e-5
    for t, r in ((l1.weights, oW1), (l1.biases, ob1), (l2.weights, oW2), (l2.biases, ob2)):
        assert rel(t.grad_numpy().reshape(r.grad.shape), r.grad) <= 1e-5
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("n_seq", [1, 3])
def test_positional_encoding_layer(orc, n_seq):
    """layers.PositionalEncoding (lib/transformer/positionalEncodingLayer.dart:29-65): x + table rows, the gradient
    passes through unchanged; table from the oracle's restatement (exponent 2i/dModel for every column)."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.layers import PositionalEncoding
    from flutter_ml_b200.tensor import Tensor
    ctx = _lib.Context()
    S, d, max_len = 7, 12, 16
    rng = np.random.default_rng(n_seq)
    x = rng.standard_normal((n_seq * S, d)).astype(np.float32)
    target = rng.standard_normal((n_seq * S, d)).astype(np.float32)
    layer = PositionalEncoding(max_len, d, seq_len=S if n_seq > 1 else 0)
    xt = Tensor(x, ctx, requires_zero_grad=True)
    out = layer(xt)
    loss = T.mseMatrix(out, Tensor(target, ctx))
    loss.backward()
    pe = orc.Ops().positional_table(max_len, d)[:S]
    want = w64(x) + np.tile(pe, (n_seq, 1))
    assert layer.parameters == []
    assert rel(out.numpy(), want) <= 1e-6
    assert rel(xt.grad_numpy(), 2 * (want - w64(target)) / want.size) <= 1e-5
    ctx.close()


def test_lm_step_with_update_on_the_side_stream_equals_the_plain_step():
    """The training step that exchanges and updates slice by slice on the side stream (head, blocks last to first,
    embedding; Adam and zeroGrad fused, under the rest of the backward pass) must leave exactly the parameters, the
    optimizer state and the cleared gradients that forward, backward, one Adam launch and zeroGrad leave
    (lib/nets/snet.dart:74-85), over several steps."""
    from flutter_ml_b200 import _lib, models, synth
    V, d, heads, dff, L, S, B = 600, 128, 2, 256, 2, 128, 2
    params = models.init_lm(4, V, d, heads, dff, L, std=0.05)
    ids, labels = synth.integers(4, 100, (B * S,), V), synth.integers(4, 101, (B * S,), V)
    res = []
    for overlap in (False, False, True):
        ctx = _lib.Context(precision=_lib.PREC_TF32)
        lm = models.TransformerLM(ctx, params, S, heads, lr=1e-3)
        d_ids, d_lab = ctx.upload(ids), ctx.upload(labels)
        losses = [float(lm.train_step(d_ids, d_lab, B * S, overlap_exchange=overlap).numpy()[0]) for _ in range(3)]
        ctx.sync()
        res.append((losses, lm.arena.values.numpy(), lm.optimizer._m.numpy(), lm.optimizer._v.numpy(), lm.arena.grads.numpy()))
        assert ctx.device_status() == 0
        ctx.close()
    (l0, w0, m0, v0, g0), (lr_, wr, mr, vr, gr), (l1, w1, m1, v1, g1) = res
    assert l0[2] < l0[0]                                     # it trains
    # Split-K weight gradients add their partial sums with atomics in no fixed order, so two runs of the SAME step differ in
    # the last bits of the gradients, and Adam turns that into full-size steps of either sign wherever a gradient is
    # mathematically zero (the key bias: softmax is invariant to a shift of the scores).  The yardstick is therefore the
    # difference between two plain runs: the overlapped step may differ from a plain run by no more than three times that.
    noise_w, noise_m, noise_v = rel(wr, w0), rel(mr, m0), rel(vr, v0)
    print(f"plain vs plain: w {noise_w:.2e} m {noise_m:.2e} v {noise_v:.2e}; overlapped vs plain: w {rel(w1, w0):.2e} "
          f"m {rel(m1, m0):.2e} v {rel(v1, v0):.2e}")
    assert np.allclose(l0, l1, rtol=1e-5) and np.allclose(l0, lr_, rtol=1e-5)
    assert rel(w1, w0) <= max(1e-4, 3 * noise_w) and rel(m1, m0) <= max(1e-4, 3 * noise_m) and rel(v1, v0) <= max(1e-4, 3 * noise_v)
    assert not g0.any() and not g1.any() and not gr.any()
