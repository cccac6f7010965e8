"""Data-parallel host logic on CPU with two gloo ranks: row sharding, id exchange, and that shard
gradients normalised by the GLOBAL count add up to the full-batch gradient."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_shard_rows_partition():
    from flutter_ml_b200 import dp
    for n, w in ((256, 8), (10, 4), (3, 4), (7, 2)):
        spans = [dp.shard_rows(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        dp.shard_rows(4, 4, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from flutter_ml_b200 import dp, synth
    from oracle import oracle
    uid = dp.broadcast_unique_id(dist, lambda: bytes(range(128)))
    assert uid == bytes(range(128))
    # tiny LM: each rank runs the oracle on its shard with the global normaliser, grads are summed
    rng = np.random.default_rng(0)
    V, d, S, B = 20, 8, 4, 4
    mk = lambda *s: rng.normal(0, 0.3, s)  # noqa: E731
    block = {"heads": [(mk(d, 4), mk(d, 4), mk(d, 4)) for _ in range(2)], "Wo": mk(d, d), "g1": np.ones(d), "be1": np.zeros(d),
             "W1": mk(d, 12), "b1": np.zeros(12), "W2": mk(12, d), "b2": np.zeros(d), "g2": np.ones(d), "be2": np.zeros(d)}
    params = {"emb": mk(V, d), "blocks": [block], "Whead": mk(d, V), "bhead": np.zeros(V)}
    ids, labels = synth.integers(0, 1, (B, S), V), synth.integers(0, 2, (B, S), V)
    r0, r1 = dp.shard_rows(B, rank, world)
    part = oracle.lm_forward_backward(ids[r0:r1], labels[r0:r1], params, B * S)
    flat = torch.tensor(np.concatenate([g.ravel() for g in part["grads"]] + [[part["loss"]]]))
    dist.all_reduce(flat)
    if rank == 0:
        full = oracle.lm_forward_backward(ids, labels, params, B * S)
        ref = np.concatenate([g.ravel() for g in full["grads"]] + [[full["loss"]]])
        out.put(float(np.abs(flat.numpy() - ref).max()))
    dist.destroy_process_group()


def test_two_rank_gloo_gradients_sum_to_full_batch():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) < 1e-12
