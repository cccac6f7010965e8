"""Timing of benchmark configurations 1, 3 and 4 at their stated sizes (config 2 is bench.py's main
line, config 5 is train_bench).  Inputs are seeded synthetic tensors; times are CUDA events on the
library's stream, averaged over `reps` steps after `warm` untimed ones."""
from __future__ import annotations

import ctypes

import numpy as np

from flutter_ml_b200 import _lib, models, synth
from flutter_ml_b200 import tensor as T
from flutter_ml_b200.tensor import Tensor


def _timed(ctx, fn, warm=2, reps=5):
    for _ in range(warm):
        fn()
    ctx.sync()
    l0 = ctx.launches
    ctx.timer_start()
    for _ in range(reps):
        fn()
    ms = ctx.timer_stop_ms() / reps
    return ms, (ctx.launches - l0) // reps


def config1_mlp(ctx):
    """MLP 784-128-64-10, batch 64, one forward + backward + SGD step."""
    mlp = models.MLP(ctx, models.init_mlp(0), lr=0.01)
    X, labels = ctx.upload(synth.uniform(0, 0, (64, 784))), ctx.upload(synth.integers(0, 1, (64,), 10))
    ms, launches = _timed(ctx, lambda: mlp.train_step(X, labels), warm=5, reps=50)
    flops = 41926656.0
    out = {"config": "C1 MLP 784-128-64-10 batch 64 fwd+bwd+SGD", "us_per_step": round(ms * 1e3, 1),
           "samples_per_s": round(64 / ms * 1e3, 1), "gflops": round(flops / ms / 1e6, 1), "launches_per_step": launches}
    # the same step recorded once as a CUDA graph and replayed (one call per step instead of ~15)
    mlp.record_step(X, labels)
    gms, _ = _timed(ctx, mlp.replay_step, warm=5, reps=200)
    out.update({"graph_us_per_step": round(gms * 1e3, 1), "graph_samples_per_s": round(64 / gms * 1e3, 1)})
    out.update(_config1_tape(ctx))
    out.update(_config1_fed(ctx, mlp))
    return out


def _feed_arms(ctx, mlp, X, y, B):
    """(prefetching feeder, blocking upload per step) in ms per step of batch B over the host arrays X, y."""
    from flutter_ml_b200.feeder import BatchFeeder
    batches = X.shape[0] // B
    feeder = BatchFeeder(ctx, [X, y], B)
    for xb, yb in feeder.batches():      # warm-up epoch
        mlp.train_step(xb, yb)
    ctx.sync()
    ctx.timer_start()
    for xb, yb in feeder.batches():
        mlp.train_step(xb, yb)
    fed_ms = ctx.timer_stop_ms() / batches
    dX, dy = ctx.empty(B, X.shape[1]), ctx.empty(B, dtype=np.int32)
    ctx.sync()
    ctx.timer_start()
    for s in range(batches):
        ctx.upload(X[B * s:B * s + B], out=dX)
        ctx.upload(y[B * s:B * s + B], out=dy)
        mlp.train_step(dX, dy)
    return fed_ms, ctx.timer_stop_ms() / batches


def _config1_fed(ctx, mlp):
    """The same step with every batch coming from HOST memory: through the prefetching feeder (staging + copy lane,
    one batch ahead) and, for comparison, with a blocking upload in front of every step the way the reference's
    binding stages its operands (lib/cuda/cudacaller.dart:32-47).  At batch 64 the step is bound by the host's
    launch rate either way; the second pair uses batches of 16384 rows (51 MB), where the copy is what is hidden."""
    X = np.concatenate([synth.uniform(0, 100 + i, (64, 784)) for i in range(200)])
    y = np.concatenate([synth.integers(0, 300 + i, (64,), 10) for i in range(200)])
    fed_ms, blk_ms = _feed_arms(ctx, mlp, X, y, 64)
    out = {"fed_us_per_step": round(fed_ms * 1e3, 1), "fed_samples_per_s": round(64 / fed_ms * 1e3, 1),
           "blocking_upload_us_per_step": round(blk_ms * 1e3, 1), "fed_h2d_bytes_per_step": 64 * 785 * 4}
    # fed + graph replay: one recorded step per device batch buffer of the feeder, replayed alternately, so a step
    # from host memory costs two library calls (events) and one graph launch
    from flutter_ml_b200.feeder import BatchFeeder
    feeder = BatchFeeder(ctx, [X, y], 64)
    for b in range(2):                   # recording runs the step once eagerly: give it defined inputs
        ctx.zero(feeder.device[b][0])
        ctx.zero(feeder.device[b][1])
    graphs = [mlp.record_step(feeder.device[b][0], feeder.device[b][1]) for b in range(2)]
    launches = mlp._graph_launches
    for _ in range(2):                   # first pass warms up, second is timed
        ctx.sync()
        ctx.timer_start()
        for s, _batch in enumerate(feeder.batches()):
            ctx.graph_launch(graphs[s % 2], launches=launches)
        fg_ms = ctx.timer_stop_ms() / len(feeder)
    out.update({"fed_graph_us_per_step": round(fg_ms * 1e3, 1), "fed_graph_samples_per_s": round(64 / fg_ms * 1e3, 1)})
    B = 16384
    X = synth.uniform(0, 500, (12 * B, 784))
    y = synth.integers(0, 501, (12 * B,), 10)
    fed_ms, blk_ms = _feed_arms(ctx, mlp, X, y, B)
    out["fed_batch16384"] = {"fed_ms_per_step": round(fed_ms, 3), "blocking_upload_ms_per_step": round(blk_ms, 3),
                             "fed_samples_per_s": round(B / fed_ms * 1e3, 1), "h2d_gbs": round(B * 785 * 4 / fed_ms / 1e6, 1)}
    return out


def _config1_tape(ctx):
    """The same step as a node list for the tape executor: three `dense` nodes + softmax cross-entropy, one library
    call per sweep (forward, backward) and one for SGD over the six parameters' flat arena."""
    from flutter_ml_b200.optimizers import ParameterArena
    from flutter_ml_b200.tape import Tape
    tp = Tape(ctx)
    P = [tp.tensor(p) for p in models.init_mlp(0)]
    h = tp.tensor(synth.uniform(0, 0, (64, 784)), requires_grad=False)
    for l, act in enumerate(("relu", "relu", None)):
        h = tp.dense(h, P[2 * l], P[2 * l + 1], act)
    tp.softmaxCrossEntropy(h, tp.ids(synth.integers(0, 1, (64,), 10)), 1.0 / 64)
    arena = ParameterArena(ctx, P)   # parameters and their gradients become slices of two flat buffers
    tp.compile()

    def step():
        tp.forward()
        tp.backward()
        ctx.call("fml_sgd_step", arena.values, arena.grads, arena.size, 0.01, 1.0)
        arena.zero_grads()
    ms, _ = _timed(ctx, step, warm=5, reps=200)
    return {"tape_us_per_step": round(ms * 1e3, 1), "tape_samples_per_s": round(64 / ms * 1e3, 1)}


def config3_encoder_block(ctx):
    """Post-LN encoder block d512 h8 dff2048, seq 256, batch 32, causal, forward + backward."""
    d, heads, dff, S, B = 512, 8, 2048, 256, 32
    from flutter_ml_b200.layers import TransformerEncoderBlock
    block = TransformerEncoderBlock(d, heads, dff, seq_len=S, causal=True, params=models.init_block(2, d, heads, dff))
    x = ctx.upload(synth.normal(2, 500, (B * S, d)))
    tgt = Tensor(ctx.upload(synth.normal(2, 501, (B * S, d))), ctx)

    def step():
        xt = Tensor(x, ctx)
        loss = T.mseMatrix(block(xt), tgt, weight=float(B))
        loss.backward()
        for p in block.parameters:
            p.grad = None
    ms, launches = _timed(ctx, step)
    flops = 1.675e11
    out = {"config": "C3 encoder block d512 h8 dff2048 S256 B32 causal fwd+bwd", "ms_per_step": round(ms, 3),
           "tflops": round(flops / ms / 1e9, 1), "sequences_per_s": round(B / ms * 1e3, 1), "launches_per_step": launches}
    # the same step recorded once as a CUDA graph and replayed (29 launches issued with one call)
    import gc
    gc.collect()
    ctx.graph_begin()
    try:
        step()
        gc.collect()                    # every buffer allocated while recording is freed while recording
    finally:
        gid = ctx.graph_end()
    if gid >= 0:
        gms, _ = _timed(ctx, lambda: ctx.graph_launch(gid), warm=3, reps=20)
        out.update({"graph_ms_per_step": round(gms, 3), "graph_tflops": round(flops / gms / 1e9, 1)})
    return out


def config4_lstm(ctx):
    """LSTM input 256, hidden 512, seq 128, batch 128, forward + BPTT (loss: mse of the last hidden state)."""
    Tn, B, I, H = 128, 128, 256, 512
    a = 1.0 / np.sqrt(512.0)
    W, b = ctx.upload(synth.uniform(3, 0, (4 * H, H + I), -a, a)), ctx.zeros(4 * H)
    x = ctx.upload(synth.normal(3, 2, (Tn * B, I)))
    target = ctx.upload(synth.normal(3, 3, (B, H)))
    d = _lib.LstmDesc()
    d.T, d.B, d.I, d.H = Tn, B, I, H
    bufs = dict(W=W, b=b, x=x, gates=ctx.empty(Tn, B, 4 * H), cells=ctx.empty(Tn + 1, B, H), hs=ctx.empty(Tn + 1, B, H),
                xproj=ctx.empty(Tn * B, 4 * H))
    for k, v in bufs.items():
        setattr(d, k, v.ptr)
    dW, db, dh, loss = ctx.zeros(4 * H, H + I), ctx.zeros(4 * H), ctx.empty(B, H), ctx.zeros(1)
    scratch = ctx.empty(Tn * B * 4 * H + 2 * B * H)
    h_last = bufs["hs"].view(Tn * B * H, (B, H))

    def step():
        ctx.check(ctx.lib.fml_lstm_fwd(ctx.h, ctypes.byref(d)))
        ctx.call("fml_mse", h_last, target, dh, loss, B * H, float(B), launches=2)
        ctx.check(ctx.lib.fml_lstm_bwd(ctx.h, ctypes.byref(d), dh.ptr, dW.ptr, db.ptr, None, scratch.ptr))
        ctx.launches += Tn + 11   # forward: regrouping, input projection, ONE recurrence kernel; backward: ONE fused launch per step + the weight-gradient products
    ms, launches = _timed(ctx, step)
    fwd_ms, _ = _timed(ctx, lambda: ctx.check(ctx.lib.fml_lstm_fwd(ctx.h, ctypes.byref(d))))
    bwd_ms, _ = _timed(ctx, lambda: ctx.check(ctx.lib.fml_lstm_bwd(ctx.h, ctypes.byref(d), dh.ptr, dW.ptr, db.ptr, None, scratch.ptr)))
    flops = 1.546e11
    return {"fwd_ms": round(fwd_ms, 3), "bwd_ms": round(bwd_ms, 3), "config": "C4 LSTM I256 H512 T128 B128 fwd+BPTT", "ms_per_step": round(ms, 3), "tflops": round(flops / ms / 1e9, 1),
            "us_per_timestep": round(ms * 1e3 / (2 * Tn), 1), "sequences_per_s": round(B / ms * 1e3, 1),
            "launches_per_step": launches}


def tiered_lstm(ctx):
    """The two-tier layer (lib/layertypes/duallstm.dart) at configuration 4's sizes: I 256, H 512, T 128, batch 128, clock
    cycle 7; forward + backward through layers.DualLSTMLayer (three products and one cell kernel per update)."""
    from flutter_ml_b200.layers import DualLSTMLayer
    I, H, Tn, B, cyc = 256, 512, 128, 128, 7
    x = Tensor(synth.normal(3, 40, (Tn, B, I)), ctx)
    target = Tensor(synth.normal(3, 41, (B, H)), ctx)
    layer = DualLSTMLayer(H, cyc, seed=3)

    def step():
        loss = T.mseMatrix(layer(x), target)
        loss.backward()
    ms, launches = _timed(ctx, step, warm=2, reps=3)
    # the same step recorded once as a CUDA graph and replayed: what is left when the host's launch calls are out of the way
    import gc
    gc.collect()
    graph_ms = None
    ctx.graph_begin()
    try:
        step()
        gc.collect()                    # every buffer allocated while recording is freed while recording
    finally:
        gid = ctx.graph_end()
    if gid >= 0:
        graph_ms, _ = _timed(ctx, lambda: ctx.graph_launch(gid), warm=2, reps=5)
    updates = Tn + sum(1 for t in range(Tn) if t > 0 and (t + 1) % cyc == 0)
    flops = 3.0 * 2 * B * 4 * H * (Tn * (2 * H + I) + (updates - Tn) * 2 * H)
    return {"config": f"DualLSTM I{I} H{H} T{Tn} B{B} cycle {cyc} fwd+bwd (next-row layer, not a BASELINE config)", "ms_per_step": round(ms, 3),
            "tflops": round(flops / ms / 1e9, 1), "us_per_update_and_direction": round(ms * 1e3 / (2 * updates), 1), "launches_per_step": launches,
            "graph_ms_per_step": round(graph_ms, 3) if graph_ms else None}


def run(ctx, only: int = 0):
    """All three configurations plus the tiered layer, or just configuration `only` (1, 3 or 4; for profiling one of them)."""
    fns = {1: config1_mlp, 3: config3_encoder_block, 4: config4_lstm, 6: tiered_lstm}
    return [fn(ctx) for k, fn in fns.items() if only in (0, k)]
