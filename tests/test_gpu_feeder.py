"""Batched data feeding: host arrays -> page-locked staging -> copy lane -> device batches, one batch ahead."""
import numpy as np
import pytest

from tests.gpu_util import rel

pytestmark = pytest.mark.gpu


def _net(seed0):
    from flutter_ml_b200.layers import DenseLayerMatrix
    from flutter_ml_b200.snet import SNetwork
    return SNetwork([DenseLayerMatrix(32, "tanh", seed=seed0), DenseLayerMatrix(16, "relu", seed=seed0 + 1),
                     DenseLayerMatrix(4, None, seed=seed0 + 2)])


def _data(n, seed):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, 24))
    Wt = rng.standard_normal((24, 4)) * 0.3
    return X, np.tanh(X @ Wt)      # float64 on purpose: the feeder narrows while it stages


def test_feeder_delivers_every_row_in_order_including_a_short_last_batch():
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.feeder import BatchFeeder
    ctx = _lib.Context()
    n, B = 1000, 96                                   # 10 full batches + one of 40
    X = np.arange(n * 7, dtype=np.float64).reshape(n, 7)
    y = (np.arange(n) % 13).astype(np.int64)
    f = BatchFeeder(ctx, [X, y], B)
    assert len(f) == 11
    for order in (None, np.random.default_rng(0).permutation(n)):
        idx = np.arange(n) if order is None else order
        seen = 0
        for s, (xb, yb) in enumerate(f.batches(order)):
            rows = min(B, n - s * B)
            assert xb.shape == (rows, 7) and yb.shape == (rows,) and yb.dtype == np.int32
            want = idx[s * B:s * B + rows]
            assert np.array_equal(xb.numpy(), X[want].astype(np.float32))
            assert np.array_equal(yb.numpy(), y[want].astype(np.int32))
            seen += rows
        assert seen == n
    assert f.h2d_bytes == 2 * n * (7 + 1) * 4
    assert len(list(BatchFeeder(ctx, [X, y], B, drop_last=True).batches())) == 10
    # two feeders walked in lock step on one context (training and validation): separate event slots
    g = BatchFeeder(ctx, [X[::-1].copy(), y[::-1].copy()], B, event_slots=52)
    for s, ((xa, ya), (xb, yb)) in enumerate(zip(f.batches(), g.batches())):
        rows = min(B, n - s * B)
        assert np.array_equal(xa.numpy(), X[s * B:s * B + rows].astype(np.float32))
        assert np.array_equal(xb.numpy(), X[::-1][s * B:s * B + rows].astype(np.float32))
        assert np.array_equal(yb.numpy(), y[::-1][s * B:s * B + rows].astype(np.int32))
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("opt_name", ["sgd", "adam"])
def test_fit_batched_equals_fit_on_uploaded_batches(opt_name):
    """Same kernels in the same order on the same rows: feeding from the host with prefetch must leave exactly the
    parameters that fit() leaves when every batch was uploaded beforehand, and report the same epoch losses."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200.optimizers import SGD, Adam
    from flutter_ml_b200.tensor import Tensor, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_FP32)
    set_default_context(ctx)
    n, B, epochs = 200, 48, 3                          # 4 full batches + one of 8
    X, Y = _data(n, 11)
    make = (lambda ps: SGD(ps, 0.05)) if opt_name == "sgd" else (lambda ps: Adam(ps, 0.01))

    a = _net(20)
    a.predict(Tensor(X[:B].astype(np.float32), ctx))
    a.compile(make(a.parameters))
    xs = [Tensor(X[s:s + B].astype(np.float32), ctx) for s in range(0, n, B)]
    ys = [Tensor(Y[s:s + B].astype(np.float32), ctx) for s in range(0, n, B)]
    hist_a = a.fit(xs, ys, epochs=epochs)

    b = _net(20)
    b.predict(Tensor(X[:B].astype(np.float32), ctx))
    b.compile(make(b.parameters))
    hist_b = b.fitBatched(X, Y, B, epochs)

    for pa, pb in zip(a.parameters, b.parameters):
        assert rel(pb.numpy(), pa.numpy()) <= 1e-6      # only sums formed with atomics may differ in the last bit
    assert np.allclose(hist_a, hist_b, rtol=1e-5)
    assert hist_b[-1] < hist_b[0]
    assert b.feeder.h2d_bytes == epochs * n * (24 + 4) * 4
    assert ctx.device_status() == 0
    ctx.close()


def test_fit_batched_with_labels_and_shuffle_follows_the_oracle(orc):
    """Integer labels + softmax cross-entropy + a seeded shuffle per epoch, against the float64 tape of the oracle
    walking the same batches."""
    from flutter_ml_b200 import _lib
    from flutter_ml_b200 import tensor as T
    from flutter_ml_b200.optimizers import SGD
    from flutter_ml_b200.tensor import Tensor, set_default_context
    ctx = _lib.Context(precision=_lib.PREC_3XTF32)
    set_default_context(ctx)
    n, B, epochs, lr, seed = 120, 40, 2, 0.1, 5
    X, _ = _data(n, 3)
    labels = np.random.default_rng(4).integers(0, 4, n)
    X32 = X.astype(np.float32)

    net = _net(30)
    net.predict(Tensor(X32[:B], ctx))
    P0 = [p.numpy().astype(np.float64) for p in net.parameters]
    net.compile(SGD(net.parameters, lr))
    hist = net.fitBatched(X, labels, B, epochs, loss=lambda out, lab: T.softmaxCrossEntropy(out, lab, 1.0 / out.shape[0]),
                          shuffle_seed=seed)

    E = orc.Engine()
    P = [orc.T(p) for p in P0]
    want_hist = []
    for epoch in range(epochs):
        order = np.random.default_rng(seed + epoch).permutation(n)
        tot = 0.0
        for s in range(0, n, B):
            idx = order[s:s + B]
            h = orc.T(X32[idx].astype(np.float64))
            for l, act in enumerate(("tanh", "relu", None)):
                h = E.dense_matrix(h, P[2 * l], P[2 * l + 1], act)
            loss = E.softmaxCrossEntropy(h, labels[idx], 1.0 / len(idx))
            loss.backward()
            for p in P:
                p.value -= lr * p.grad
                p.grad[...] = 0
            tot += float(np.ravel(loss.value)[0])
        want_hist.append(tot / (n // B))
    for p, w in zip(net.parameters, P):
        assert rel(p.numpy(), w.value) <= 2e-5
    assert np.allclose(hist, want_hist, rtol=1e-4)
    assert ctx.device_status() == 0
    ctx.close()


def test_fed_graph_replay_equals_fed_eager_steps():
    """One recorded step per device batch buffer of the feeder, replayed alternately while the feeder refills the
    other buffer: same parameters as the eager step over the same batches."""
    from flutter_ml_b200 import _lib, models, synth
    from flutter_ml_b200.feeder import BatchFeeder
    ctx = _lib.Context()
    n, B = 64 * 9, 64
    X = np.concatenate([synth.uniform(0, 100 + i, (64, 784)) for i in range(9)])
    y = np.concatenate([synth.integers(0, 300 + i, (64,), 10) for i in range(9)])
    finals = []
    for use_graph in (False, True):
        mlp = models.MLP(ctx, models.init_mlp(0), lr=0.01)
        feeder = BatchFeeder(ctx, [X, y], B)
        for b in range(2):
            ctx.zero(feeder.device[b][0])
            ctx.zero(feeder.device[b][1])
        if use_graph:
            graphs = [mlp.record_step(feeder.device[b][0], feeder.device[b][1]) for b in range(2)]
        else:
            for b in range(2):              # the eager step that recording runs first
                mlp.train_step(feeder.device[b][0], feeder.device[b][1])
        for s, (xb, yb) in enumerate(feeder.batches()):
            if use_graph:
                ctx.graph_launch(graphs[s % 2])
            else:
                mlp.train_step(xb, yb)
        finals.append(mlp.arena.values.numpy())
    assert np.isfinite(finals[0]).all()
    assert rel(finals[1], finals[0]) <= 1e-6
    assert ctx.device_status() == 0
    ctx.close()
