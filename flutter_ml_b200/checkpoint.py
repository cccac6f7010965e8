"""Checkpoints of parameters and optimizer state (`fml_checkpoint_save` / `fml_checkpoint_load`).

The reference has no serialisation; this is the step either side of the training loop.  A checkpoint is a
set of named fp32 device buffers plus a step counter.  `state_of` collects what a training run needs to
resume: the flat parameter arena (or the parameter tensors one by one) and the optimizer's state buffers.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

from . import _lib


def _arrays(named: Dict[str, "_lib.DeviceArray"]):
    n = len(named)
    names = (C.c_char_p * n)(*[k.encode() for k in named])
    bufs = (_lib.fp * n)(*[v.ptr for v in named.values()])
    sizes = (_lib.i64 * n)(*[v.size for v in named.values()])
    return n, names, bufs, sizes


def save(ctx, path: str, named: Dict[str, "_lib.DeviceArray"], step: int = 0) -> None:
    n, names, bufs, sizes = _arrays(named)
    ctx.check(ctx.lib.fml_checkpoint_save(ctx.h, path.encode(), int(step), n, C.cast(names, _lib.fp), C.cast(bufs, _lib.fp),
                                          C.cast(sizes, _lib.fp)))


def load(ctx, path: str, named: Dict[str, "_lib.DeviceArray"]) -> int:
    """Restore the listed buffers (a subset of the file is fine) and return the stored step counter."""
    n, names, bufs, sizes = _arrays(named)
    step = _lib.i64(0)
    ctx.check(ctx.lib.fml_checkpoint_load(ctx.h, path.encode(), C.byref(step), n, C.cast(names, _lib.fp), C.cast(bufs, _lib.fp),
                                          C.cast(sizes, _lib.fp)))
    return step.value


def state_of(optimizer) -> Dict[str, "_lib.DeviceArray"]:
    """Named buffers of an optimizer from `flutter_ml_b200.optimizers` and of the parameters it updates."""
    out = {}
    if optimizer.arena is not None:
        out["parameters"] = optimizer.arena.values
    else:
        for i, p in enumerate(optimizer.parameters):
            out[f"parameter.{i}"] = p.value
    states = []
    if hasattr(optimizer, "_m"):
        states = [("m", optimizer._m), ("v", optimizer._v)]
    elif hasattr(optimizer, "_state"):
        states = [(f"s{k + 1}", s) for k, s in enumerate(optimizer._state)]
    for name, s in states:
        if isinstance(s, list):
            for i, a in enumerate(s):
                out[f"optimizer.{name}.{i}"] = a
        else:
            out[f"optimizer.{name}"] = s
    return out


def save_training_state(ctx, path: str, optimizer) -> None:
    save(ctx, path, state_of(optimizer), step=getattr(optimizer, "_t", 0))


def load_training_state(ctx, path: str, optimizer) -> None:
    optimizer._t = load(ctx, path, state_of(optimizer))
