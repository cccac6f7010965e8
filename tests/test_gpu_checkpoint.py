"""Checkpoint round trips through the C ABI: bit-exact restore, resume equals uninterrupted training,
and every malformed-file case is refused before device memory is touched."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ctx():
    from flutter_ml_b200 import _lib
    c = _lib.Context(precision=_lib.PREC_FP32)
    yield c
    c.close()


def test_round_trip_is_bit_exact_and_subsets_load(ctx, tmp_path):
    from flutter_ml_b200 import checkpoint
    rng = np.random.default_rng(0)
    # one entry larger than two 16 MiB staging chunks, one odd-sized, one single float
    host = {"big": rng.standard_normal(9_000_001).astype(np.float32), "odd": rng.standard_normal(12345).astype(np.float32),
            "one": np.array([3.25], np.float32)}
    dev = {k: ctx.upload(v) for k, v in host.items()}
    path = str(tmp_path / "a.ckpt")
    checkpoint.save(ctx, path, dev, step=77)
    assert os.path.getsize(path) == 8 + 8 + 4 + sum(4 + len(k) + 8 + 4 for k in host) + 4 * sum(v.size for v in host.values())
    assert not os.path.exists(path + ".tmp")
    for v in dev.values():
        ctx.zero(v)
    assert checkpoint.load(ctx, path, dev) == 77
    for k in host:
        assert np.array_equal(dev[k].numpy().ravel(), host[k])
    only = {"odd": ctx.zeros(12345)}
    assert checkpoint.load(ctx, path, only) == 77
    assert np.array_equal(only["odd"].numpy(), host["odd"])


def test_bad_files_are_refused_without_touching_device_memory(ctx, tmp_path):
    from flutter_ml_b200 import _lib, checkpoint
    a = ctx.upload(np.arange(1000, dtype=np.float32))
    path = str(tmp_path / "b.ckpt")
    checkpoint.save(ctx, path, {"a": a}, step=1)
    keep = ctx.upload(np.full(1000, 7.0, np.float32))
    with pytest.raises(_lib.FmlError, match="no entry named"):
        checkpoint.load(ctx, path, {"missing": keep})
    with pytest.raises(_lib.FmlError, match="size mismatch"):
        checkpoint.load(ctx, path, {"a": ctx.zeros(999)})
    raw = bytearray(open(path, "rb").read())
    raw[-5] ^= 0x40                       # flip one payload bit
    open(path, "wb").write(raw)
    with pytest.raises(_lib.FmlError, match="checksum mismatch"):
        checkpoint.load(ctx, path, {"a": keep})
    assert np.all(keep.numpy() == 7.0)    # nothing was overwritten
    open(path, "wb").write(raw[:40])      # truncated
    with pytest.raises(_lib.FmlError):
        checkpoint.load(ctx, path, {"a": keep})
    open(path, "wb").write(b"not a checkpoint at all")
    with pytest.raises(_lib.FmlError, match="not a checkpoint"):
        checkpoint.load(ctx, path, {"a": keep})
    with pytest.raises(_lib.FmlError, match="cannot open"):
        checkpoint.load(ctx, str(tmp_path / "nope.ckpt"), {"a": keep})


@pytest.mark.parametrize("opt_name", ["Adam", "AMSGrad", "SGDMomentum"])
def test_resume_equals_uninterrupted_training(tmp_path, opt_name):
    """Four optimizer steps in one run == two steps, save, fresh process state, load, two more steps."""
    from flutter_ml_b200 import _lib, checkpoint, models, optimizers, synth
    X, labels = synth.uniform(0, 0, (64, 784)), synth.integers(0, 1, (64,), 10)
    path = str(tmp_path / "train.ckpt")

    def make():
        ctx = _lib.Context(precision=_lib.PREC_FP32)
        mlp = models.MLP(ctx, models.init_mlp(0), lr=0.01)
        opt = getattr(optimizers, opt_name)(mlp.parameters, 0.01, arena=mlp.arena)
        return ctx, mlp, opt

    def steps(ctx, mlp, opt, n):
        from flutter_ml_b200.tensor import Tensor, softmaxCrossEntropy
        dX, dl = ctx.upload(X), ctx.upload(labels)
        for _ in range(n):
            softmaxCrossEntropy(mlp.forward(Tensor(dX, ctx)), dl, 1.0 / 64).backward()
            opt.step()
            opt.zeroGrad()

    ctx, mlp, opt = make()
    steps(ctx, mlp, opt, 4)
    straight = mlp.arena.values.numpy().copy()
    ctx.close()

    ctx, mlp, opt = make()
    steps(ctx, mlp, opt, 2)
    checkpoint.save_training_state(ctx, path, opt)
    ctx.close()

    ctx, mlp, opt = make()
    checkpoint.load_training_state(ctx, path, opt)
    assert opt._t == 2
    steps(ctx, mlp, opt, 2)
    assert np.array_equal(mlp.arena.values.numpy(), straight)
    ctx.close()
