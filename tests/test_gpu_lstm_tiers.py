"""The tiered recurrent layers on the GPU (layers.MultiTierLSTMLayer, layers.DualLSTMLayer over fml_lstm_cell_fwd/bwd and
the library's products) against the oracle's composition of the reference's vector operations
(lib/layertypes/multilstm.dart:111-178, lib/layertypes/duallstm.dart:98-175)."""
import numpy as np
import pytest

from tests.gpu_util import rel

pytestmark = pytest.mark.gpu
w64 = lambda x: np.ascontiguousarray(x, dtype=np.float64)  # noqa: E731


def test_lstm_cell_kernels(orc):
    """fml_lstm_cell_fwd / _bwd alone: gate blocks f | i | c~ | o, the reference's activation rules (sigmoid, tanh with its
    overflow rule, derivatives from the outputs), with and without incoming dc, writing and accumulating dc_prev."""
    from flutter_ml_b200 import _lib
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    rng = np.random.default_rng(3)
    B, H = 7, 20
    pre, cp = rng.standard_normal((B, 4 * H)).astype(np.float32) * 2, rng.standard_normal((B, H)).astype(np.float32)
    dh, dc = rng.standard_normal((B, H)).astype(np.float32), rng.standard_normal((B, H)).astype(np.float32)
    d_pre, d_cp = ctx.upload(pre), ctx.upload(cp)
    gates, c, h = ctx.empty(B, 4 * H), ctx.empty(B, H), ctx.empty(B, H)
    ctx.call("fml_lstm_cell_fwd", d_pre, d_cp, gates, c, h, B, H)
    sg = lambda z: 1 / (1 + np.exp(-z))  # noqa: E731
    p = w64(pre)
    f, i, g, o = sg(p[:, :H]), sg(p[:, H:2 * H]), np.tanh(p[:, 2 * H:3 * H]), sg(p[:, 3 * H:])
    c_ref = f * w64(cp) + i * g
    h_ref = o * np.tanh(c_ref)
    assert rel(gates.numpy(), np.concatenate([f, i, g, o], 1)) <= 1e-6
    assert rel(c.numpy(), c_ref) <= 1e-6 and rel(h.numpy(), h_ref) <= 1e-6
    for use_dc in (True, False):
        for acc in (0, 1):
            dpre, dcp0 = ctx.empty(B, 4 * H), rng.standard_normal((B, H)).astype(np.float32)
            dcp = ctx.upload(dcp0)
            ctx.call("fml_lstm_cell_bwd", gates, d_cp, c, ctx.upload(dh), ctx.upload(dc) if use_dc else None, dpre, dcp, acc, B, H)
            tc = np.tanh(c_ref)
            dct = (w64(dc) if use_dc else 0.0) + w64(dh) * o * (1 - tc * tc)
            ref = np.concatenate([dct * w64(cp) * f * (1 - f), dct * g * i * (1 - i), dct * i * (1 - g * g), w64(dh) * tc * o * (1 - o)], 1)
            assert rel(dpre.numpy(), ref) <= 2e-6
            assert rel(dcp.numpy(), dct * f + (w64(dcp0) if acc else 0.0)) <= 2e-6
    assert ctx.device_status() == 0
    ctx.close()


def test_lstm_cell_kernels_reject_bad_arguments():
    """NULL buffers and non-positive or oversize extents come back as an error status with a message; the context stays
    usable (the reference's FFI surface returns nothing at all, lib/cuda/cudacaller.dart:25-60)."""
    from flutter_ml_b200 import _lib
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    B, H = 4, 8
    pre, cp = ctx.zeros(B, 4 * H), ctx.zeros(B, H)
    gates, c, h = ctx.empty(B, 4 * H), ctx.empty(B, H), ctx.empty(B, H)
    for bad in ((None, cp, gates, c, h, B, H), (pre, cp, gates, c, None, B, H), (pre, cp, gates, c, h, 0, H), (pre, cp, gates, c, h, B, -1),
                (pre, cp, gates, c, h, 1 << 20, 1 << 20)):
        with pytest.raises(RuntimeError):
            ctx.call("fml_lstm_cell_fwd", *bad)
    with pytest.raises(RuntimeError):
        ctx.call("fml_lstm_cell_bwd", gates, cp, c, None, None, None, cp, 0, B, H)      # no dpre
    ctx.call("fml_lstm_cell_fwd", pre, cp, gates, c, h, B, H)                            # still works
    assert np.allclose(h.numpy(), 0.0) and ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("kind,cycles,B,Tn,H,I,prec", [
    ("multi", [3, 2], 4, 14, 32, 12, 1), ("multi", [2], 1, 9, 16, 5, 1), ("multi", [2, 2, 2], 3, 17, 8, 4, 2),
    ("dual", [4], 3, 13, 64, 8, 1), ("dual", [1], 2, 6, 16, 4, 2), ("multi", [3, 2], 5, 14, 32, 12, 0)])
def test_tiered_lstm_layers(orc, kind, cycles, B, Tn, H, I, prec):
    """Last hidden state of tier 0, loss, every parameter gradient (in the reference's order, tier by tier) and the input
    gradient against the oracle, sequence by sequence; 3xTF32 and FP32 at 1e-5 / 2e-5, TF32 at the bounds of a chain of
    truncating products."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.layers import DualLSTMLayer, MultiTierLSTMLayer
    from flutter_ml_b200.tensor import Tensor
    ctx = _lib.Context(precision=prec)
    rng = np.random.default_rng(100 * B + Tn + H)
    n = len(cycles) + 1
    combs = [H + (n - 1) * H + I] + [2 * H] * (n - 1)
    Ws = [rng.uniform(-1, 1, (4 * H, cb)).astype(np.float32) * np.float32(np.sqrt(1.0 / cb)) for cb in combs]
    bs = [rng.uniform(-0.1, 0.1, 4 * H).astype(np.float32) for _ in range(n)]
    x = rng.standard_normal((Tn, B, I)).astype(np.float32)
    target = rng.standard_normal((B, H)).astype(np.float32)
    layer = (DualLSTMLayer(H, cycles[0], weights=Ws, biases=bs) if kind == "dual" else MultiTierLSTMLayer(H, cycles, weights=Ws, biases=bs))
    xin = Tensor(x[:, 0, :] if B == 1 else x, ctx)
    xin.zeroGrad()                                   # ask for the input gradient
    out = layer(xin)
    assert out.shape == (B, H) and len(layer.parameters) == 8 * n
    loss = T.mseMatrix(out, Tensor(target, ctx), weight=float(B))       # = sum over sequences of mse(h_b, target_b)
    loss.backward()
    h_ref, loss_ref = np.zeros((B, H)), 0.0
    dW_ref, db_ref, dx_ref = [np.zeros_like(w64(w)) for w in Ws], [np.zeros(4 * H) for _ in range(n)], np.zeros((Tn, B, I))
    for b in range(B):
        h_b, l_b, dWs, dbs, dx_b = orc.tiered_lstm_fwd_bwd(w64(x[:, b, :]), [w64(w) for w in Ws], [w64(v) for v in bs], cycles, w64(target[b]),
                                                            dual=(kind == "dual"))
        h_ref[b], loss_ref = h_b, loss_ref + l_b
        for i in range(n):
            dW_ref[i] += dWs[i]
            db_ref[i] += dbs[i]
        dx_ref[:, b, :] = dx_b
    t_out, t_grad = {0: (2e-3, 5e-3), 1: (1e-5, 2e-5), 2: (1e-5, 2e-5)}[prec]
    errs = {"h": rel(out.numpy(), h_ref), "dx": rel(xin.grad_numpy().reshape(Tn, B, I), dx_ref)}
    for i in range(n):
        for g in range(4):
            Wg, bg = layer.parameters[8 * i + 2 * g], layer.parameters[8 * i + 2 * g + 1]
            assert np.array_equal(Wg.numpy(), Ws[i][g * H:(g + 1) * H]) and np.array_equal(bg.numpy(), bs[i][g * H:(g + 1) * H])
        errs[f"dW{i}"] = rel(np.concatenate([layer.parameters[8 * i + 2 * g].grad_numpy() for g in range(4)]), dW_ref[i])
        errs[f"db{i}"] = rel(np.concatenate([layer.parameters[8 * i + 2 * g + 1].grad_numpy() for g in range(4)]), db_ref[i])
    print(f"PARITY tiered-lstm {kind} {cycles} B{B} T{Tn} H{H} prec{prec}: " + " ".join(f"{k} {v:.1e}" for k, v in errs.items()))
    assert errs["h"] <= t_out and abs(loss.numpy()[0] - loss_ref) <= 2 * t_out * abs(loss_ref)
    for k, v in errs.items():
        if k != "h":
            assert v <= t_grad, (k, v)
    assert ctx.device_status() == 0
    ctx.close()


def test_snetwork_with_a_dual_lstm_layer_trains():
    """SNetwork([DualLSTMLayer, DenseLayerMatrix]) with fit(), the shape of the reference's demo
    (lib/layertypes/duallstm.dart:180-300): the loss goes down."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.layers import DenseLayerMatrix, DualLSTMLayer
    from flutter_ml_b200.optimizers import Adam
    from flutter_ml_b200.snet import SNetwork
    from flutter_ml_b200.tensor import Tensor, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    set_default_context(ctx)
    rng = np.random.default_rng(1)
    t = np.arange(400) * 0.3
    wave = np.sin(t) + 0.5 * np.sin(t / 7.0)
    xs = [Tensor(wave[i:i + 14].reshape(14, 1).astype(np.float32), ctx) for i in range(0, 60, 3)]
    ys = [Tensor(np.array([[wave[i + 14]]], dtype=np.float32), ctx) for i in range(0, 60, 3)]
    net = SNetwork([DualLSTMLayer(12, 7, seed=2), DenseLayerMatrix(1, None, seed=3)])
    net.predict(xs[0])
    net.compile(Adam(net.parameters, 0.02))
    hist = net.fit(xs, ys, epochs=12)
    assert hist[-1] < 0.5 * hist[0]
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("B,Tn,H,W,k", [(1, 4, 7, 7, 3), (3, 5, 9, 6, 3), (2, 3, 8, 8, 5)])
def test_conv_lstm_layer(orc, B, Tn, H, W, k):
    """layers.ConvLSTMLayer (lib/layertypes/convlstmLayer.dart:37-159): last hidden map, loss, the twelve parameter
    gradients in the reference's order and the input gradient against the oracle, sequence by sequence."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.layers import ConvLSTMLayer
    from flutter_ml_b200.tensor import Tensor
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    rng = np.random.default_rng(10 * B + Tn + k)
    Kx = (rng.uniform(-1, 1, (4, k, k)) / k).astype(np.float32)
    Kh = (rng.uniform(-1, 1, (4, k, k)) / k).astype(np.float32)
    bias = rng.uniform(-0.1, 0.1, (4, H, W)).astype(np.float32)
    x = rng.standard_normal((Tn, B, H, W)).astype(np.float32)
    target = rng.standard_normal((B, H, W)).astype(np.float32)
    layer = ConvLSTMLayer(8, k, kernels_x=Kx, kernels_h=Kh, biases=bias)
    xin = Tensor(x[:, 0] if B == 1 else x, ctx)
    xin.zeroGrad()
    out = layer(xin)
    assert out.shape == ((H, W) if B == 1 else (B, H, W)) and len(layer.parameters) == 12
    loss = T.mseMatrix(out, Tensor(target[0] if B == 1 else target, ctx), weight=float(B))   # = sum over sequences of mseMatrix
    loss.backward()
    h_ref, loss_ref = np.zeros((B, H, W)), 0.0
    dKx_ref, dKh_ref, db_ref, dx_ref = np.zeros((4, k, k)), np.zeros((4, k, k)), np.zeros((4, H, W)), np.zeros((Tn, B, H, W))
    for b in range(B):
        h_b, l_b, a, c_, d_, e_ = orc.conv_lstm_fwd_bwd(w64(x[:, b]), w64(Kx), w64(Kh), w64(bias), w64(target[b]))
        h_ref[b], loss_ref = h_b, loss_ref + l_b
        dKx_ref += a
        dKh_ref += c_
        db_ref += d_
        dx_ref[:, b] = e_
    P = layer.parameters
    for g in range(4):
        assert np.array_equal(P[3 * g].numpy(), Kx[g]) and np.array_equal(P[3 * g + 1].numpy(), Kh[g]) and np.array_equal(P[3 * g + 2].numpy(), bias[g])
    errs = {"h": rel(out.numpy().reshape(B, H, W), h_ref), "dx": rel(xin.grad_numpy().reshape(Tn, B, H, W), dx_ref),
            "dKx": rel(np.stack([P[3 * g].grad_numpy() for g in range(4)]), dKx_ref),
            "dKh": rel(np.stack([P[3 * g + 1].grad_numpy() for g in range(4)]), dKh_ref),
            "db": rel(np.stack([P[3 * g + 2].grad_numpy() for g in range(4)]), db_ref)}
    print(f"PARITY conv-lstm B{B} T{Tn} {H}x{W} k{k}: " + " ".join(f"{n} {v:.1e}" for n, v in errs.items()))
    assert abs(loss.numpy()[0] - loss_ref) <= 1e-5 * abs(loss_ref)
    for n, v in errs.items():
        assert v <= 1e-5, (n, v)
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("grains,B,Tn,H,I,final_len,prec", [([7, 4], 1, 60, 16, 4, 7, 1), ([3, 2], 3, 31, 32, 8, 4, 1), ([4], 2, 9, 8, 4, 5, 2),
                                                            ([2, 2, 2], 2, 40, 16, 4, 3, 2), ([3, 2], 4, 50, 32, 8, 6, 0)])
def test_chained_scale_layer(orc, grains, B, Tn, H, I, final_len, prec):
    """layers.GeneralizedChainedScaleLayer (lib/layertypes/trendmodelLayer.dart:42-218): last hidden state of level 0, loss,
    every LSTM and aggregation parameter gradient (in the reference's order) and the input gradient against the oracle,
    sequence by sequence."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.layers import GeneralizedChainedScaleLayer
    from flutter_ml_b200.tensor import Tensor
    ctx = _lib.Context(precision=prec)
    rng = np.random.default_rng(7 * B + Tn + H)
    n = len(grains) + 1
    Z = H + I
    Ws = [(rng.uniform(-1, 1, (4 * H, Z)) * np.sqrt(1.0 / Z)).astype(np.float32) for _ in range(n)]
    bs = [rng.uniform(-0.1, 0.1, 4 * H).astype(np.float32) for _ in range(n)]
    aWs = [(rng.uniform(-1, 1, (I, g * I)) * np.sqrt(1.0 / (g * I))).astype(np.float32) for g in grains]
    abs_ = [rng.uniform(-0.1, 0.1, I).astype(np.float32) for _ in grains]
    x = rng.standard_normal((B, Tn, I)).astype(np.float32)
    target = rng.standard_normal((B, H)).astype(np.float32)
    layer = GeneralizedChainedScaleLayer(H, grains, final_len, lstm_weights=Ws, lstm_biases=bs, agg_weights=aWs, agg_biases=abs_)
    xin = Tensor(x[0] if B == 1 else x, ctx)
    xin.zeroGrad()
    out = layer(xin)
    assert out.shape == ((H,) if B == 1 else (B, H)) and len(layer.parameters) == 8 * n + 2 * len(grains)
    loss = T.mseMatrix(out, Tensor(target[0] if B == 1 else target, ctx), weight=float(B))
    loss.backward()
    h_ref, loss_ref = np.zeros((B, H)), 0.0
    dW_ref, db_ref = [np.zeros((4 * H, Z)) for _ in range(n)], [np.zeros(4 * H) for _ in range(n)]
    daW_ref, dab_ref, dx_ref = [np.zeros_like(w64(w)) for w in aWs], [np.zeros(I) for _ in grains], np.zeros((B, Tn, I))
    for b in range(B):
        h_b, l_b, dWs, dbs, daWs, dabs, dx_b = orc.chained_scale_fwd_bwd(w64(x[b]), [w64(w) for w in Ws], [w64(v) for v in bs], [w64(w) for w in aWs],
                                                                         [w64(v) for v in abs_], grains, final_len, w64(target[b]))
        h_ref[b], loss_ref, dx_ref[b] = h_b, loss_ref + l_b, dx_b
        for i in range(n):
            dW_ref[i] += dWs[i]
            db_ref[i] += dbs[i]
        for i in range(len(grains)):
            daW_ref[i] += daWs[i]
            dab_ref[i] += dabs[i]
    P = layer.parameters
    errs = {"h": rel(out.numpy().reshape(B, H), h_ref), "dx": rel(xin.grad_numpy().reshape(B, Tn, I), dx_ref)}
    for i in range(n):
        errs[f"dW{i}"] = rel(np.concatenate([P[8 * i + 2 * g].grad_numpy() for g in range(4)]), dW_ref[i])
        errs[f"db{i}"] = rel(np.concatenate([P[8 * i + 2 * g + 1].grad_numpy() for g in range(4)]), db_ref[i])
    for i in range(len(grains)):
        errs[f"daW{i}"] = rel(P[8 * n + 2 * i].grad_numpy(), daW_ref[i])
        errs[f"dab{i}"] = rel(P[8 * n + 2 * i + 1].grad_numpy(), dab_ref[i])
    print(f"PARITY chained-scale {grains} B{B} T{Tn} H{H} prec{prec}: " + " ".join(f"{k} {v:.1e}" for k, v in errs.items()))
    # TF32: the gradient of the highest aggregation level has passed through three LSTM loops (up to 26 steps, two
    # truncating products each) and two aggregation products; the operand truncation biases every product by the same
    # sign, so the error grows with the depth of the chain (measured 5.6e-3 at the top, 9e-4 at the bottom).
    t_out, t_grad = {0: (2e-3, 1e-2), 1: (1e-5, 2e-5), 2: (1e-5, 2e-5)}[prec]
    assert errs["h"] <= t_out and abs(loss.numpy()[0] - loss_ref) <= 2 * t_out * abs(loss_ref)
    for k, v in errs.items():
        if k != "h":
            assert v <= t_grad, (k, v)
    assert ctx.device_status() == 0
    ctx.close()
