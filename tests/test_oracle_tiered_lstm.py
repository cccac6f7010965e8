"""The oracle's restatement of the tiered recurrent layers (lib/layertypes/multilstm.dart, duallstm.dart), checked on the
CPU: its analytic gradients against central differences of its own loss, and the one place where the two layers differ.
The reference holds no fixed vectors for these layers (its demos print unseeded results), so this pins the restatement's
backward sweep to its forward pass, not to reference outputs."""
import numpy as np
import pytest


def _case(rng, H, I, cycles):
    n = len(cycles) + 1
    Ws = [rng.standard_normal((4 * H, H + (n - 1) * H + I)) * 0.5] + [rng.standard_normal((4 * H, 2 * H)) * 0.5 for _ in range(n - 1)]
    bs = [rng.standard_normal(4 * H) * 0.1 for _ in range(n)]
    return Ws, bs


@pytest.mark.parametrize("cycles,dual,Tn", [([2, 3], False, 13), ([3], True, 10), ([], False, 5)])
def test_tiered_lstm_gradients_match_central_differences(orc, cycles, dual, Tn):
    rng = np.random.default_rng(len(cycles) * 10 + Tn)
    H, I = 3, 2
    Ws, bs = _case(rng, H, I, cycles)
    x, tgt = rng.standard_normal((Tn, I)), rng.standard_normal(H)
    h, loss, dWs, dbs, dx = orc.tiered_lstm_fwd_bwd(x, Ws, bs, cycles, tgt, dual=dual)
    assert h.shape == (H,) and np.isfinite(loss)

    def L(Ws_, bs_, x_):
        return orc.tiered_lstm_fwd_bwd(x_, Ws_, bs_, cycles, tgt, dual=dual)[1]
    eps = 1e-6
    for tier in range(len(Ws)):
        for _ in range(4):
            idx = (int(rng.integers(4 * H)), int(rng.integers(Ws[tier].shape[1])))
            Wp, Wm = [w.copy() for w in Ws], [w.copy() for w in Ws]
            Wp[tier][idx] += eps
            Wm[tier][idx] -= eps
            num = (L(Wp, bs, x) - L(Wm, bs, x)) / (2 * eps)
            assert abs(dWs[tier][idx] - num) <= 1e-7 + 1e-5 * abs(num)
        j = int(rng.integers(4 * H))
        bp, bm = [b.copy() for b in bs], [b.copy() for b in bs]
        bp[tier][j] += eps
        bm[tier][j] -= eps
        num = (L(Ws, bp, x) - L(Ws, bm, x)) / (2 * eps)
        assert abs(dbs[tier][j] - num) <= 1e-7 + 1e-5 * abs(num)
    for _ in range(4):
        idx = (int(rng.integers(Tn)), int(rng.integers(I)))
        xp, xm = x.copy(), x.copy()
        xp[idx] += eps
        xm[idx] -= eps
        num = (L(Ws, bs, xp) - L(Ws, bs, xm)) / (2 * eps)
        assert abs(dx[idx] - num) <= 1e-7 + 1e-5 * abs(num)


def test_dual_layer_skips_the_first_step_of_a_unit_clock(orc):
    """With a clock cycle of 1 the multi-tier layer updates its higher tier at step 0 (multilstm.dart:155), the dual layer
    does not (`i > 0`, duallstm.dart:145); for longer cycles the two rules coincide."""
    rng = np.random.default_rng(5)
    H, I, Tn = 3, 2, 6
    Ws, bs = _case(rng, H, I, [1])
    x, tgt = rng.standard_normal((Tn, I)), rng.standard_normal(H)
    h_m = orc.tiered_lstm_fwd_bwd(x, Ws, bs, [1], tgt, dual=False)[0]
    h_d = orc.tiered_lstm_fwd_bwd(x, Ws, bs, [1], tgt, dual=True)[0]
    assert np.max(np.abs(h_m - h_d)) > 1e-6
    Ws, bs = _case(rng, H, I, [3])
    h_m = orc.tiered_lstm_fwd_bwd(x, Ws, bs, [3], tgt, dual=False)[0]
    h_d = orc.tiered_lstm_fwd_bwd(x, Ws, bs, [3], tgt, dual=True)[0]
    assert np.array_equal(h_m, h_d)


def test_a_single_tier_is_the_plain_lstm(orc):
    """No clock cycles = one tier on [h, x_t]: the reference's LSTMLayer (lstmLayer.dart:112-150), which the oracle
    restates separately (lstm_fwd_bwd)."""
    rng = np.random.default_rng(6)
    H, I, Tn = 4, 3, 7
    W = rng.standard_normal((4, H, H + I)) * 0.4
    b = rng.standard_normal((4, H)) * 0.1
    x, tgt = rng.standard_normal((1, Tn, I)), rng.standard_normal((1, H))
    h_ref, loss_ref, dW_ref, db_ref = orc.Ops().lstm_fwd_bwd(W, b, x, tgt)
    h, loss, dWs, dbs, _ = orc.tiered_lstm_fwd_bwd(x[0], [W.reshape(4 * H, H + I)], [b.reshape(4 * H)], [], tgt[0])
    assert np.allclose(h, h_ref[0], rtol=1e-12, atol=1e-14) and abs(loss - loss_ref) <= 1e-12 * abs(loss_ref)
    assert np.allclose(dWs[0].reshape(4, H, H + I), dW_ref, rtol=1e-10, atol=1e-14)
    assert np.allclose(dbs[0].reshape(4, H), db_ref, rtol=1e-10, atol=1e-14)


def test_conv_lstm_gradients_match_central_differences(orc):
    """The oracle's ConvLSTM (lib/layertypes/convlstmLayer.dart:107-159, composed from its conv2d / addMatrix / sigmoidMatrix /
    tanhMatrix / elementWiseMultiplyMatrix): analytic gradients against central differences of its own loss."""
    rng = np.random.default_rng(1)
    Tn, H, W, k = 4, 5, 6, 3
    Kx, Kh = rng.standard_normal((4, k, k)) * 0.4, rng.standard_normal((4, k, k)) * 0.4
    b, x, tgt = rng.standard_normal((4, H, W)) * 0.1, rng.standard_normal((Tn, H, W)), rng.standard_normal((H, W))
    h, loss, dKx, dKh, db, dx = orc.conv_lstm_fwd_bwd(x, Kx, Kh, b, tgt)
    assert h.shape == (H, W) and np.isfinite(loss)
    arrs, grads = {"Kx": Kx, "Kh": Kh, "b": b, "x": x}, {"Kx": dKx, "Kh": dKh, "b": db, "x": dx}
    eps = 1e-6
    for name, arr in arrs.items():
        for _ in range(5):
            pos = tuple(int(rng.integers(n)) for n in arr.shape)
            vals = []
            for sgn in (+1, -1):
                a2 = {k_: v.copy() for k_, v in arrs.items()}
                a2[name][pos] += sgn * eps
                vals.append(orc.conv_lstm_fwd_bwd(a2["x"], a2["Kx"], a2["Kh"], a2["b"], tgt)[1])
            num = (vals[0] - vals[1]) / (2 * eps)
            assert abs(grads[name][pos] - num) <= 1e-7 + 1e-5 * abs(num), (name, pos)


@pytest.mark.parametrize("grains,Tn,final_len", [([3, 2], 31, 4), ([4], 9, 5), ([2, 2, 2], 40, 3)])
def test_chained_scale_gradients_match_central_differences(orc, grains, Tn, final_len):
    """The oracle's GeneralizedChainedScaleLayer (lib/layertypes/trendmodelLayer.dart:134-204): analytic gradients against
    central differences of its own loss, for the LSTM weights of every tier, the aggregation weights of every level and
    the input (old rows reach the loss only through the summaries)."""
    rng = np.random.default_rng(len(grains) + Tn)
    H, I = 3, 2
    n = len(grains) + 1
    Ws = [rng.standard_normal((4 * H, H + I)) * 0.5 for _ in range(n)]
    bs = [rng.standard_normal(4 * H) * 0.1 for _ in range(n)]
    aWs = [rng.standard_normal((I, g * I)) * 0.5 for g in grains]
    abs_ = [rng.standard_normal(I) * 0.1 for _ in grains]
    x, tgt = rng.standard_normal((Tn, I)), rng.standard_normal(H)
    h, loss, dWs, dbs, daWs, dabs, dx = orc.chained_scale_fwd_bwd(x, Ws, bs, aWs, abs_, grains, final_len, tgt)
    assert h.shape == (H,) and np.isfinite(loss)

    def L(**kw):
        a = dict(Ws=Ws, bs=bs, aWs=aWs, abs_=abs_, x=x)
        a.update(kw)
        return orc.chained_scale_fwd_bwd(a["x"], a["Ws"], a["bs"], a["aWs"], a["abs_"], grains, final_len, tgt)[1]
    eps = 1e-6

    def check(name, arrs, grads, i, pos):
        p_, m_ = [a.copy() for a in arrs], [a.copy() for a in arrs]
        p_[i][pos] += eps
        m_[i][pos] -= eps
        num = (L(**{name: p_}) - L(**{name: m_})) / (2 * eps)
        assert abs(grads[i][pos] - num) <= 2e-9 + 1e-4 * abs(num), (name, i, pos, grads[i][pos], num)
    for i in range(n):
        for _ in range(3):
            check("Ws", Ws, dWs, i, (int(rng.integers(4 * H)), int(rng.integers(H + I))))
        check("bs", bs, dbs, i, (int(rng.integers(4 * H)),))
    for i in range(len(grains)):
        for _ in range(3):
            check("aWs", aWs, daWs, i, (int(rng.integers(I)), int(rng.integers(grains[i] * I))))
        check("abs_", abs_, dabs, i, (int(rng.integers(I)),))
    for _ in range(5):
        pos = (int(rng.integers(Tn)), int(rng.integers(I)))
        xp, xm = x.copy(), x.copy()
        xp[pos] += eps
        xm[pos] -= eps
        num = (L(x=xp) - L(x=xm)) / (2 * eps)
        assert abs(dx[pos] - num) <= 2e-9 + 1e-4 * abs(num), (pos, dx[pos], num)
