"""fml_tape_run: whole autograd tapes submitted with one call per sweep, against the oracle's tape
(same node list, float64, reference accumulation semantics)."""
import math

import numpy as np
import pytest

from tests.gpu_util import rel

pytestmark = pytest.mark.gpu


def w64(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32), dtype=np.float64)


@pytest.fixture()
def fp32_ctx():
    from flutter_ml_b200 import _lib
    c = _lib.Context(precision=_lib.PREC_FP32)
    yield c
    c.close()


def test_matvec_sum_demo_known_answer(fp32_ctx):
    """The reference's printed demo (tensor.dart:1359-1376): M = [[1,2],[3,4]], v = [10,20], s = sum(M.v).
    Values derived by hand: M.v = [50, 110], s = 160, dM = [[10,20],[10,20]], dv = [4, 6]."""
    from flutter_ml_b200.tape import Tape
    tp = Tape(fp32_ctx)
    M, v = tp.tensor([[1, 2], [3, 4]]), tp.tensor([10, 20])
    y = tp.matVecMul(M, v)
    s = tp.sum(y)
    tp.forward()
    tp.backward()
    assert y.numpy().ravel().tolist() == [50.0, 110.0]
    assert float(s.numpy()[0, 0]) == 160.0
    assert M.grad_numpy().tolist() == [[10.0, 20.0], [10.0, 20.0]]
    assert v.grad_numpy().ravel().tolist() == [4.0, 6.0]
    # gradients of leaves accumulate over sweeps until zeroGrad (tensor.dart:77-91)
    tp.backward()
    assert v.grad_numpy().ravel().tolist() == [8.0, 12.0]
    v.zeroGrad()
    assert v.grad_numpy().ravel().tolist() == [0.0, 0.0]


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("prec,tol", [(2, 2e-6), (1, 2e-5), (0, 2e-3)])   # chains of three products: model-level bounds
def test_mlp_config1_as_a_tape(orc, fused, prec, tol):
    """Config 1's network as a node list: matMul + addMatrixAndVector + relu_matrix per layer (or the fused
    `dense` node), softmax cross-entropy; logits, loss and all six gradients against the oracle."""
    from flutter_ml_b200 import _lib, models, synth
    from flutter_ml_b200.tape import Tape
    ctx = _lib.Context(precision=prec)
    params = models.init_mlp(0)
    X = synth.uniform(0, 0, (64, 784))
    labels = synth.integers(0, 1, (64,), 10)
    ref = orc.mlp_step(w64(X), labels, [w64(p) for p in params], lr=0.01, omp=True)
    tp = Tape(ctx)
    P = [tp.tensor(p) for p in params]
    h = tp.tensor(X, requires_grad=False)
    for l, act in enumerate(("relu", "relu", None)):
        W, b = P[2 * l], P[2 * l + 1]
        if fused:
            h = tp.dense(h, W, b, act)
        else:
            h = tp.addMatrixAndVector(tp.matMul(h, W), b)
            h = tp.reluMatrix(h) if act else h
    logits = h
    loss = tp.softmaxCrossEntropy(logits, tp.ids(labels), 1.0 / X.shape[0])
    tp.forward()
    tp.backward()
    assert rel(logits.numpy(), ref["logits"]) <= tol
    assert abs(float(loss.numpy()[0, 0]) - ref["loss"]) <= max(tol, 1e-6) * abs(ref["loss"])
    if prec != 0:
        assert np.array_equal(logits.numpy().argmax(1), ref["logits"].argmax(1))
    gtol = 5e-2 if prec == 0 else 5 * tol   # TF32: ReLU gates of near-zero pre-activations may flip
    for p, g in zip(P, ref["grads"]):
        assert rel(p.grad_numpy().reshape(g.shape), g) <= gtol
    assert len(tp) == (4 if fused else 9)
    ctx.close()


def _attention_block(E, x, heads, Wo, g, be, target, dk, softmax):
    outs = []
    for Wq, Wk, Wv in heads:
        Q, K, V = E.matMul(x, Wq), E.matMul(x, Wk), E.matMul(x, Wv)
        s = E.scaleMatrix(E.matMul(Q, E.transpose(K)), 1 / math.sqrt(dk))
        outs.append(E.matMul(softmax(s), V))
    attn = E.matMul(E.concatenateMatricesByColumn(outs), Wo)
    y = E.layerNorm(E.addMatrix(x, attn), g, be)
    return E.mseMatrix(y, target), y


@pytest.mark.parametrize("causal", [False, True])
def test_attention_block_as_a_tape(orc, fp32_ctx, causal):
    """Two attention heads written with the reference's own node vocabulary (matMul, transpose, scale_matrix,
    softmax_matrix, concat_matrix_col, add_matrix, layer_norm, mse_matrix; singleHeadAttentionLayer.dart:70-89,
    multiHeadAttentionLayer.dart:72-84): x is consumed seven times, so its gradient tests the fan-in +=."""
    from flutter_ml_b200.tape import Tape
    S, d, dk = 48, 64, 32
    rng = np.random.default_rng(5 + causal)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    x, target = f(S, d), f(S, d)
    heads = [(f(d, dk) * 0.2, f(d, dk) * 0.2, f(d, dk) * 0.2) for _ in range(2)]
    Wo, g, be = f(2 * dk, d) * 0.2, 1 + 0.1 * f(d), 0.1 * f(d)

    E = orc.Engine()
    ox, oh = orc.T(w64(x)), [tuple(orc.T(w64(w)) for w in h) for h in heads]
    oWo, og, obe = orc.T(w64(Wo)), orc.T(w64(g)), orc.T(w64(be))
    oloss, oy = _attention_block(E, ox, oh, oWo, og, obe, orc.T(w64(target)), dk, lambda s: E.softmaxMatrix(s, causal))
    oloss.backward()

    tp = Tape(fp32_ctx)
    tx, th = tp.tensor(x), [tuple(tp.tensor(w) for w in h) for h in heads]
    tWo, tg, tbe = tp.tensor(Wo), tp.tensor(g), tp.tensor(be)
    tloss, ty = _attention_block(tp, tx, th, tWo, tg, tbe, tp.tensor(target, requires_grad=False), dk,
                                 lambda s: tp.softmaxMatrix(s, S if causal else 0))
    tp.forward()
    tp.backward()
    assert rel(ty.numpy(), oy.value) <= 2e-6
    assert abs(float(tloss.numpy()[0, 0]) - float(oloss.value)) <= 2e-6 * float(oloss.value)
    pairs = [(tx, ox), (tWo, oWo), (tg, og), (tbe, obe)] + [(a, b) for hh, oo in zip(th, oh) for a, b in zip(hh, oo)]
    for t, o in pairs:
        assert rel(t.grad_numpy().reshape(o.grad.shape), o.grad) <= 2e-5


def test_lstm_cell_in_vector_form_as_a_tape(orc, fp32_ctx):
    """LSTMLayer.forward exactly as the reference writes it (lstmLayer.dart:112-150): concat_vector, four
    matVecMul + add_vector + sigmoid/tanh per step, multiply_vector, three time steps; 18 nodes per step."""
    from flutter_ml_b200.tape import Tape
    I, H, Tn = 12, 20, 3
    rng = np.random.default_rng(9)
    f = lambda *s: (rng.standard_normal(s) * 0.4).astype(np.float32)
    Ws, bs = [f(H, H + I) for _ in range(4)], [f(H) for _ in range(4)]
    xs, target = [f(I) for _ in range(Tn)], f(H)

    def run(E, mk, vec):
        W, b = [mk(w) for w in Ws], [mk(v) for v in bs]
        h, c = mk(np.zeros(H, np.float32)), mk(np.zeros(H, np.float32))
        for x in xs:
            z = E.concatenate(h, mk(x))
            gate = lambda k, fn: fn(vec.add(E.matVecMul(W[k], z), b[k]))
            f_t, i_t, c_t = gate(0, vec.sigmoid), gate(1, vec.sigmoid), gate(2, vec.tanh)
            c = vec.add(E.elementWiseMultiply(f_t, c), E.elementWiseMultiply(i_t, c_t))
            o_t = gate(3, vec.sigmoid)
            h = E.elementWiseMultiply(o_t, vec.tanh(c))
        return vec.mse(h, mk(target)), h, W, b

    E = orc.Engine()

    class OV:   # the oracle's unary ops take any shape
        add, sigmoid, tanh = staticmethod(E.addMatrix), staticmethod(E.sigmoidMatrix), staticmethod(E.tanhMatrix)
        mse = staticmethod(E.mseMatrix)
    oloss, oh, oW, ob = run(E, lambda a: orc.T(w64(a)), OV)
    oloss.backward()

    tp = Tape(fp32_ctx)

    class TV:
        add, sigmoid, tanh, mse = tp.addVector, tp.sigmoid, tp.vectorTanh, tp.mse
    tloss, th, tW, tb = run(tp, tp.tensor, TV)
    tp.forward()
    tp.backward()
    assert len(tp) == 18 * Tn + 1
    assert rel(th.numpy().ravel(), oh.value) <= 2e-6
    assert abs(float(tloss.numpy()[0, 0]) - float(oloss.value)) <= 2e-6 * float(oloss.value)
    for t, o in list(zip(tW, oW)) + list(zip(tb, ob)):
        assert rel(t.grad_numpy().reshape(o.grad.shape), o.grad) <= 1e-5


def test_embedding_and_other_activations_on_the_tape(orc, fp32_ctx):
    from flutter_ml_b200.tape import Tape
    V, d, n = 30, 16, 25
    rng = np.random.default_rng(12)
    table = rng.standard_normal((V, d)).astype(np.float32)
    ids = rng.integers(0, V, n).astype(np.int32)
    target = rng.standard_normal((n, d)).astype(np.float32)
    E = orc.Engine()
    ot = orc.T(w64(table))
    oe = E.embedding(ot, ids)
    o = E.act2(8, E.act2(7, E.act2(6, E.act2(5, oe, 0.1), 0.7)))
    ol = E.mseMatrix(E.elementWiseMultiply(o, oe), orc.T(w64(target)))
    ol.backward()
    tp = Tape(fp32_ctx)
    tt_ = tp.tensor(table)
    te = tp.embeddingLookup(tt_, tp.ids(ids))
    t = tp.mish(tp.swish(tp.elu(tp.leakyRelu(te, 0.1), 0.7)))
    tl = tp.mseMatrix(tp.elementWiseMultiply(t, te), tp.tensor(target, requires_grad=False))
    tp.forward()
    tp.backward()
    assert abs(float(tl.numpy()[0, 0]) - float(ol.value)) <= 2e-6 * float(ol.value)
    assert rel(tt_.grad_numpy(), ot.grad) <= 1e-5


def test_tape_rejects_unknown_kinds_and_missing_buffers(fp32_ctx):
    import ctypes as C
    from flutter_ml_b200 import _lib
    ops = (_lib.Op * 1)()
    buf = fp32_ctx.zeros(16)
    ops[0].kind, ops[0].rows, ops[0].cols, ops[0].out = 99, 4, 4, buf.ptr
    assert fp32_ctx.lib.fml_tape_run(fp32_ctx.h, ops, 1, 0) == -1
    assert b"unknown kind" in fp32_ctx.lib.fml_last_error(fp32_ctx.h)
    ops[0].kind = 1   # matMul without inputs
    assert fp32_ctx.lib.fml_tape_run(fp32_ctx.h, ops, 1, 0) == -1
    assert fp32_ctx.lib.fml_tape_run(fp32_ctx.h, ops, 1, 7) == -1      # direction
    assert fp32_ctx.lib.fml_tape_run(fp32_ctx.h, ops, 1, 1) == -1      # backward without gout
    assert fp32_ctx.lib.fml_tape_run(fp32_ctx.h, None, 0, 0) == 0      # empty tape


def test_tape_sweeps_replay_as_a_cuda_graph(fp32_ctx):
    """Forward + backward of a tape recorded into a CUDA graph: the replay reproduces the eager sweep."""
    from flutter_ml_b200.tape import Tape
    rng = np.random.default_rng(2)
    X, W, b, Tt = (rng.standard_normal(s).astype(np.float32) for s in ((64, 128), (128, 96), (96,), (64, 96)))
    tp = Tape(fp32_ctx)
    tx, tW, tb = tp.tensor(X, requires_grad=False), tp.tensor(W), tp.tensor(b)
    loss = tp.mseMatrix(tp.dense(tx, tW, tb, "tanh"), tp.tensor(Tt, requires_grad=False))
    tp.forward()
    tp.backward()
    eager_loss, eager_gW = loss.numpy().copy(), tW.grad_numpy().copy()
    tW.zeroGrad(), tb.zeroGrad()
    fp32_ctx.sync()
    fp32_ctx.graph_begin()
    tp.forward()
    tp.backward()
    gid = fp32_ctx.graph_end()
    tW.zeroGrad(), tb.zeroGrad()
    fp32_ctx.graph_launch(gid)
    assert np.array_equal(loss.numpy(), eager_loss)
    assert np.allclose(tW.grad_numpy(), eager_gW, rtol=1e-6, atol=1e-7)


def test_tape_training_step_with_flat_parameter_arena(orc):
    """forward, backward, SGD over one flat arena, zeroGrad - the order of SNetwork.fit (lib/nets/snet.dart:74-85) -
    for two steps: parameters against two oracle steps."""
    from flutter_ml_b200 import _lib, models, synth
    from flutter_ml_b200.optimizers import ParameterArena
    from flutter_ml_b200.tape import Tape
    ctx = _lib.Context(precision=_lib.PREC_3XTF32)
    params = models.init_mlp(0)
    X, labels = synth.uniform(0, 0, (64, 784)), synth.integers(0, 1, (64,), 10)
    ref = [w64(p) for p in params]
    for _ in range(2):
        ref = orc.mlp_step(w64(X), labels, ref, lr=0.05, omp=True)["params"]
    tp = Tape(ctx)
    P = [tp.tensor(p) for p in params]
    h = tp.tensor(X, requires_grad=False)
    for l, act in enumerate(("relu", "relu", None)):
        h = tp.dense(h, P[2 * l], P[2 * l + 1], act)
    tp.softmaxCrossEntropy(h, tp.ids(labels), 1.0 / 64)
    arena = ParameterArena(ctx, P)
    for _ in range(2):
        tp.forward()
        tp.backward()
        ctx.call("fml_sgd_step", arena.values, arena.grads, arena.size, 0.05, 1.0)
        arena.zero_grads()
    for p, r in zip(P, ref):
        assert rel(p.numpy().reshape(r.shape), r) <= 1e-5
    ctx.close()


def test_multi_tier_lstm_variant_as_a_tape(orc, fp32_ctx):
    """MultiTierLSTMLayer.forward (lib/layertypes/multilstm.dart:100-150): tier 0 sees [h_0, c_1, x_t] every
    step, tier 1 sees [h_1, h_0] every second step.  With two tiers this is also DualLSTMLayer.forward
    (lib/layertypes/duallstm.dart:98-184: lower tier on [lh, hc, x_t], higher tier on [hh, lh] every
    `lowerTierClockCycle` steps, output = final lh).  The variant needs no kernel of its own: it is a list of the
    same vector-form nodes, so it runs on the tape executor as it stands."""
    from flutter_ml_b200.tape import Tape
    I, H, Tn, cycle = 3, 10, 4, 2
    rng = np.random.default_rng(31)
    f = lambda *s: (rng.standard_normal(s) * 0.4).astype(np.float32)
    sizes = [H + H + I, H + H]       # combined input of tier 0 and tier 1
    Ws = [[f(H, n) for _ in range(4)] for n in sizes]
    bs = [[f(H) for _ in range(4)] for _ in sizes]
    xs, target = [f(I) for _ in range(Tn)], f(H)

    def run(E, mk, vec):
        W = [[mk(w) for w in tier] for tier in Ws]
        b = [[mk(v) for v in tier] for tier in bs]
        h = [mk(np.zeros(H, np.float32)) for _ in sizes]
        c = [mk(np.zeros(H, np.float32)) for _ in sizes]

        def step(z, c_prev, t):
            gate = lambda k, fn: fn(vec.add(E.matVecMul(W[t][k], z), b[t][k]))
            f_t, i_t, c_t = gate(0, vec.sigmoid), gate(1, vec.sigmoid), gate(2, vec.tanh)
            c_next = vec.add(E.elementWiseMultiply(f_t, c_prev), E.elementWiseMultiply(i_t, c_t))
            return E.elementWiseMultiply(gate(3, vec.sigmoid), vec.tanh(c_next)), c_next
        for g, x in enumerate(xs):
            h[0], c[0] = step(E.concatenate(E.concatenate(h[0], c[1]), mk(x)), c[0], 0)
            if (g + 1) % cycle == 0:
                h[1], c[1] = step(E.concatenate(h[1], h[0]), c[1], 1)
        return vec.mse(h[0], mk(target)), h[0], [w for tier in W for w in tier] + [v for tier in b for v in tier]

    E = orc.Engine()

    class OV:
        add, sigmoid, tanh = staticmethod(E.addMatrix), staticmethod(E.sigmoidMatrix), staticmethod(E.tanhMatrix)
        mse = staticmethod(E.mseMatrix)
    oloss, oh, oparams = run(E, lambda a: orc.T(w64(a)), OV)
    oloss.backward()
    tp = Tape(fp32_ctx)

    class TV:
        add, sigmoid, tanh, mse = tp.addVector, tp.sigmoid, tp.vectorTanh, tp.mse
    tloss, th, tparams = run(tp, tp.tensor, TV)
    tp.forward()
    tp.backward()
    assert rel(th.numpy().ravel(), oh.value) <= 2e-6
    assert abs(float(tloss.numpy()[0, 0]) - float(oloss.value)) <= 2e-6 * float(oloss.value)
    for t, o in zip(tparams, oparams):
        assert rel(t.grad_numpy().reshape(o.grad.shape), o.grad) <= 1e-5


def test_chained_scale_lstm_variant_as_a_tape(orc, fp32_ctx):
    """GeneralizedChainedScaleLayer.forward (lib/layertypes/trendmodelLayer.dart:134-204): each aggregation level
    turns chunks of `grain` consecutive vectors into one summary tanh(W_agg . concat(chunk) + b_agg); then one LSTM
    loop per tier, from the coarsest to the finest, each starting from the hidden state the coarser tier ended with
    (cell state restarts at zero), the finest tier over the last `final_len` raw steps.  Again only vector-form
    nodes: the executor runs it as it stands."""
    from flutter_ml_b200.tape import Tape
    I, H, steps, grains, final_len = 6, 6, 8, [2, 2], 3          # the context vector has the hidden size
    tiers = len(grains) + 1
    rng = np.random.default_rng(47)
    f = lambda *s: (rng.standard_normal(s) * 0.4).astype(np.float32)
    aggW, aggB = [f(I, g * I) for g in grains], [f(I) for _ in grains]
    Ws = [[f(H, H + I) for _ in range(4)] for _ in range(tiers)]
    bs = [[f(H) for _ in range(4)] for _ in range(tiers)]
    xs, target = [f(I) for _ in range(steps)], f(H)

    def run(E, mk, vec):
        aW, aB = [mk(w) for w in aggW], [mk(v) for v in aggB]
        W = [[mk(w) for w in tier] for tier in Ws]
        b = [[mk(v) for v in tier] for tier in bs]
        raw = [mk(x) for x in xs]
        tier_inputs, level = [raw[len(raw) - final_len:]], raw
        for i, g in enumerate(grains):
            nxt = []
            for j in range(0, len(level) - g + 1, g):
                flat = level[j]
                for v in level[j + 1:j + g]:
                    flat = E.concatenate(flat, v)
                nxt.append(vec.tanh(vec.add(E.matVecMul(aW[i], flat), aB[i])))
            tier_inputs.append(nxt)
            level = nxt
        h = mk(np.zeros(H, np.float32))
        for t in range(tiers - 1, -1, -1):
            seq = tier_inputs[t][-(final_len if t == 0 else 10):]
            c = mk(np.zeros(H, np.float32))
            for x in seq:
                z = E.concatenate(h, x)
                gate = lambda k, fn: fn(vec.add(E.matVecMul(W[t][k], z), b[t][k]))
                f_t, i_t, c_t = gate(0, vec.sigmoid), gate(1, vec.sigmoid), gate(2, vec.tanh)
                c = vec.add(E.elementWiseMultiply(f_t, c), E.elementWiseMultiply(i_t, c_t))
                h = E.elementWiseMultiply(gate(3, vec.sigmoid), vec.tanh(c))
        params = aW + aB + [w for tier in W for w in tier] + [v for tier in b for v in tier]
        return vec.mse(h, mk(target)), h, params

    E = orc.Engine()

    class OV:
        add, sigmoid, tanh = staticmethod(E.addMatrix), staticmethod(E.sigmoidMatrix), staticmethod(E.tanhMatrix)
        mse = staticmethod(E.mseMatrix)
    oloss, oh, oparams = run(E, lambda a: orc.T(w64(a)), OV)
    oloss.backward()
    tp = Tape(fp32_ctx)

    class TV:
        add, sigmoid, tanh, mse = tp.addVector, tp.sigmoid, tp.vectorTanh, tp.mse
    tloss, th, tparams = run(tp, tp.tensor, TV)
    tp.forward()
    tp.backward()
    assert rel(th.numpy().ravel(), oh.value) <= 2e-6
    assert abs(float(tloss.numpy()[0, 0]) - float(oloss.value)) <= 2e-6 * float(oloss.value)
    for t, o in zip(tparams, oparams):
        assert rel(t.grad_numpy().reshape(o.grad.shape), o.grad) <= 1e-5


@pytest.mark.parametrize("padding,kh,kw", [("valid", 3, 3), ("same", 3, 3), ("same", 5, 5), ("valid", 2, 4)])
def test_conv2d_on_the_tape(orc, fp32_ctx, padding, kh, kw):
    """conv2d + addScalarToMatrix nodes (tensor.dart:765-833, 711-737) against the oracle, gradients of image,
    kernel and scalar bias; the image feeds two convolutions, so its gradient also tests the += of the rule."""
    from flutter_ml_b200.tape import Tape
    rng = np.random.default_rng(kh * 10 + kw)
    x, k1, k2, bias = (rng.standard_normal(s).astype(np.float32) for s in ((13, 17), (kh, kw), (kh, kw), (1, 1)))
    E = orc.Engine()
    ox, ok1, ok2, ob = orc.T(w64(x)), orc.T(w64(k1)), orc.T(w64(k2)), orc.T(w64(bias[0, 0]))
    oo = E.addMatrix(E.addScalarToMatrix(E.conv2d(ox, ok1, padding), ob), E.conv2d(ox, ok2, padding))
    ol = E.mseMatrix(oo, orc.T(np.zeros_like(oo.value)))
    ol.backward()
    tp = Tape(fp32_ctx)
    tx, tk1, tk2, tb = tp.tensor(x), tp.tensor(k1), tp.tensor(k2), tp.tensor(bias)
    to = tp.addMatrix(tp.addScalarToMatrix(tp.conv2d(tx, tk1, padding), tb), tp.conv2d(tx, tk2, padding))
    tl = tp.mseMatrix(to, tp.tensor(np.zeros(to.shape, np.float32), requires_grad=False))
    tp.forward()
    tp.backward()
    assert to.shape == oo.value.shape
    assert rel(to.numpy(), oo.value) <= 2e-6
    for t, o in ((tx, ox), (tk1, ok1), (tk2, ok2), (tb, ob)):
        assert rel(t.grad_numpy().reshape(np.shape(o.grad)), o.grad) <= 1e-5


def test_conv_lstm_cell_as_a_tape(orc, fp32_ctx):
    """A ConvLSTM cell (lib/layertypes/convlstmLayer.dart:94-127) over two frames, written with the nodes it is made
    of: eight 'same' conv2d per step, add_matrix with a frame-shaped bias, sigmoid_matrix / tanh_matrix,
    multiply_matrix.  (The reference passes (kernel, frame) to conv2d in that file; the frame is the image here.)"""
    from flutter_ml_b200.tape import Tape
    Hh, Ww, k, Tn = 7, 9, 3, 2
    rng = np.random.default_rng(17)
    f = lambda *s: (rng.standard_normal(s) * 0.5).astype(np.float32)
    Kx, Kh, bs = [f(k, k) for _ in range(4)], [f(k, k) for _ in range(4)], [f(Hh, Ww) * 0.1 for _ in range(4)]
    frames, target = [f(Hh, Ww) for _ in range(Tn)], f(Hh, Ww)

    def run(E, mk, sig, tanh):
        kx, kh, b = [mk(a) for a in Kx], [mk(a) for a in Kh], [mk(a) for a in bs]
        h, c = mk(np.zeros((Hh, Ww), np.float32)), mk(np.zeros((Hh, Ww), np.float32))
        for fr in frames:
            x = mk(fr)
            gate = lambda q, fn: fn(E.addMatrix(E.addMatrix(E.conv2d(x, kx[q], "same"), E.conv2d(h, kh[q], "same")), b[q]))
            f_t, i_t, c_t = gate(0, sig), gate(1, sig), gate(2, tanh)
            c = E.addMatrix(E.elementWiseMultiply(f_t, c), E.elementWiseMultiply(i_t, c_t))
            h = E.elementWiseMultiply(gate(3, sig), tanh(c))
        return E.mseMatrix(h, mk(target)), h, kx + kh + b

    E = orc.Engine()
    oloss, oh, oparams = run(E, lambda a: orc.T(w64(a)), E.sigmoidMatrix, E.tanhMatrix)
    oloss.backward()
    tp = Tape(fp32_ctx)
    tloss, th, tparams = run(tp, tp.tensor, tp.sigmoidMatrix, tp.tanhMatrix)
    tp.forward()
    tp.backward()
    assert rel(th.numpy(), oh.value) <= 2e-6
    for t, o in zip(tparams, oparams):
        assert rel(t.grad_numpy(), o.grad) <= 2e-5


@pytest.mark.parametrize("causal", [False, True])
def test_fused_attention_node_on_the_tape(orc, causal):
    """The `attention` node (one fused kernel for all heads) inside a tape: projections by matMul, the node, the
    output projection and an mse loss, against the oracle's per-head chain (multiHeadAttentionLayer.dart:72-84)."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.tape import Tape
    ctx = _lib.Context(precision=_lib.PREC_3XTF32)   # the surrounding products near-exact; the node itself is TF32
    S, d, H, dk = 128, 96, 2, 64
    rng = np.random.default_rng(3 + causal)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    x, target = f(S, d), f(S, d)
    Wq, Wk, Wv, Wo = f(d, H * dk) * 0.1, f(d, H * dk) * 0.1, f(d, H * dk) * 0.1, f(H * dk, d) * 0.1
    E = orc.Engine()
    ox, oWo = orc.T(w64(x)), orc.T(w64(Wo))
    oheads = [tuple(orc.T(w64(W[:, h * dk:(h + 1) * dk])) for W in (Wq, Wk, Wv)) for h in range(H)]
    oy = E.multi_head(ox, oheads, oWo, causal)
    E.mseMatrix(oy, orc.T(w64(target))).backward()
    tp = Tape(ctx)
    tx, tq, tk, tv, tWo = tp.tensor(x), tp.tensor(Wq), tp.tensor(Wk), tp.tensor(Wv), tp.tensor(Wo)
    att = tp.attention(tp.matMul(tx, tq), tp.matMul(tx, tk), tp.matMul(tx, tv), S, 1 / math.sqrt(dk), causal)
    ty = tp.matMul(att, tWo)
    tp.mseMatrix(ty, tp.tensor(target, requires_grad=False))
    tp.forward()
    tp.backward()
    assert ctx.device_status() == 0
    assert rel(ty.numpy(), oy.value) <= 2e-3
    assert rel(tx.grad_numpy(), ox.grad) <= 5e-3 and rel(tWo.grad_numpy(), oWo.grad) <= 5e-3
    for h in range(H):
        for t, o in zip((tq, tk, tv), oheads[h]):
            assert rel(t.grad_numpy()[:, h * dk:(h + 1) * dk], o.grad) <= 5e-3
    ctx.close()
