"""Data-parallel training step of benchmark configuration 5, timed for bench.py.

6-layer post-LN transformer (d_model 1024, 16 heads, FFN 4096, seq 512, vocab 32000), global batch 256
sequences sharded over the ranks, causal attention, softmax cross-entropy over all tokens, Adam
(lr 1e-3), fp32 NCCL all-reduce of the 141 M-parameter gradient arena every step (slice by slice under the
backward pass, each slice's Adam update right behind its exchange).  Token ids and labels come from pinned
host memory every step and the loss is read back every step, so the figure is end to end.
Environment overrides (for quick checks): FML_TRAIN_LAYERS, FML_TRAIN_BATCH.
"""
from __future__ import annotations

import os

import numpy as np

from flutter_ml_b200 import _lib, dp, models, synth

CFG = dict(vocab=32000, d_model=1024, heads=16, dff=4096, layers=6, seq=512, batch=256, lr=1e-3, seed=4)


def flops_per_token(c) -> float:
    """Forward flops per token of the dense products: QKV, QK^T, PV (full S x S), Wo, FFN, head; x3 for fwd+bwd."""
    d, f, S, V = c["d_model"], c["dff"], c["seq"], c["vocab"]
    per_layer = 2 * d * 3 * d + 2 * S * d + 2 * S * d + 2 * d * d + 2 * d * f + 2 * f * d
    return c["layers"] * per_layer + 2 * d * V


def allreduce_bandwidth(ctx, world, barrier, max_over_ranks, n_floats=64 << 20, reps=5):
    """Bus bandwidth of the gradient exchange on its own: fml_dp_allreduce_sum over 256 MB, CUDA events, max over
    ranks; bus bandwidth = 2 (N-1)/N x bytes / time, the figure NCCL's own tests quote."""
    if world == 1:
        return None
    buf = ctx.zeros(n_floats)
    for _ in range(2):
        ctx.call("fml_dp_allreduce_sum", buf, n_floats)
    barrier()
    ctx.timer_start()
    for _ in range(reps):
        ctx.call("fml_dp_allreduce_sum", buf, n_floats)
    ms = max_over_ranks(ctx.timer_stop_ms()) / reps
    buf.free()
    return {"bytes": n_floats * 4, "ms": round(ms, 4), "busbw_gbs": round(2 * (world - 1) / world * n_floats * 4 / ms / 1e6, 1),
            "nvlink_peer_copy_gbs_measured_on_this_pool": 770.0}


def run(ctx, rank, world, barrier, max_over_ranks, steps=20, warmup=3):
    import torch.distributed as dist
    c = dict(CFG)
    c["layers"] = int(os.environ.get("FML_TRAIN_LAYERS", c["layers"]))
    c["batch"] = int(os.environ.get("FML_TRAIN_BATCH", c["batch"]))
    dp.init_data_parallel(ctx, dist if world > 1 else None, rank, world, device="cuda")
    params = models.init_lm(c["seed"], c["vocab"], c["d_model"], c["heads"], c["dff"], c["layers"], std=0.02)
    lm = models.TransformerLM(ctx, params, c["seq"], c["heads"], lr=c["lr"], rank=rank, world=world)
    del params
    r0, r1 = dp.shard_rows(c["batch"], rank, world)
    n_local = (r1 - r0) * c["seq"]
    n_global = c["batch"] * c["seq"]
    off = r0 * c["seq"]
    h_ids, h_lab = ctx.pinned((n_local,), np.int32), ctx.pinned((n_local,), np.int32)
    h_ids[...] = synth.integers(c["seed"], 100, (n_local,), c["vocab"], offset=off)
    h_lab[...] = synth.integers(c["seed"], 101, (n_local,), c["vocab"], offset=off)
    d_ids, d_lab = ctx.empty(n_local, dtype=np.int32), ctx.empty(n_local, dtype=np.int32)
    h_loss = ctx.pinned((1,), np.float32)
    losses = []

    def step():
        ctx.upload_async(h_ids, d_ids)
        ctx.upload_async(h_lab, d_lab)
        loss = lm.train_step(d_ids, d_lab, n_global)
        if world > 1:
            ctx.call("fml_dp_allreduce_sum", loss.value, 1)
        ctx.download_into(loss.value, h_loss)   # synchronises: the step's result is on the host
        losses.append(float(h_loss[0]))

    # The first step starts from identical parameters on every rank count, so its loss and the parameters it leaves
    # must agree between N = 1, 2, 4, 8 up to the summation order of the exchange (fp32).
    step()
    dp_check = {"loss_step1": losses[0], **lm.check_values()}
    for _ in range(max(warmup - 1, 0)):
        step()
    barrier()
    launches0 = ctx.launches
    ctx.timer_start()
    for _ in range(steps):
        step()
    ms = ctx.timer_stop_ms()
    barrier()
    ms = max_over_ranks(ms) / steps
    flops = 3.0 * flops_per_token(c) * n_global
    out = {"metric": "training_samples_per_s", "value": round(c["batch"] / ms * 1e3, 2), "unit": "sequences/s",
           "ms_per_step": round(ms, 2), "steps": steps, "warmup": warmup, "n_gpus": world,
           "tflops": round(flops / ms / 1e9, 1), "allreduce_bytes_per_step": int(lm.arena.size) * 4 if world > 1 else 0,
           "params": int(sum(p.value.size for p in lm.parameters)),
           "loss_first": losses[0], "loss_last": losses[-1], "gpu_launches_per_step": (ctx.launches - launches0) // steps,
           "h2d_bytes_per_step": 2 * n_local * 4, "d2h_bytes_per_step": 4, "dp_check": dp_check,
           "config": {"workload": "data-parallel transformer LM step (fwd+bwd+all-reduce+Adam)", **c,
                      "parallelism": f"dp{world}", "scaling": "strong (global batch fixed)"}}
    del lm
    bw = allreduce_bandwidth(ctx, world, barrier, max_over_ranks)
    if bw:
        out["allreduce"] = bw
    return out
