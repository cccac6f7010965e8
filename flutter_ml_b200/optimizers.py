"""Optimizers with the reference's interface (lib/optimizers/optimizers.dart:43-67):
`parameters`, `learningRate`, `step()`, `zeroGrad()`.

Parameters may be packed into one `ParameterArena` (values, grads and optimizer state each a
single contiguous buffer); `step()` is then one kernel launch for the whole model and the
data-parallel exchange one all-reduce.  Unpacked parameters are updated tensor by tensor.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np

from .tensor import Tensor


class ParameterArena:
    """Moves the given parameter tensors into one flat value buffer and one flat grad buffer
    (each tensor becomes a view at a 16-byte aligned offset)."""

    def __init__(self, ctx, parameters: List[Tensor]):
        self.ctx, self.parameters = ctx, parameters
        offs, total = [], 0
        for p in parameters:
            offs.append(total)
            total += (p.value.size + 3) & ~3
        self.size = total
        self.values, self.grads = ctx.zeros(total), ctx.zeros(total)
        for p, o in zip(parameters, offs):
            view = self.values.view(o, p.value.shape)
            ctx.copy(view, p.value)
            p.value = view
            p.grad = self.grads.view(o, p.value.shape)
        self.offsets = offs

    def zero_grads(self):
        self.ctx.zero(self.grads)


class Optimizer:
    def __init__(self, parameters: List[Tensor], learningRate: float, arena: Optional[ParameterArena] = None):
        self.parameters, self.learningRate, self.arena = parameters, learningRate, arena

    def zeroGrad(self):
        """optimizers.dart:62-66."""
        if self.arena is not None:
            self.arena.zero_grads()
        else:
            for p in self.parameters:
                p.zeroGrad()

    def step(self):
        raise NotImplementedError


class SGD(Optimizer):
    """w -= lr * g (lib/optimizers/sgd.dart:24-42)."""

    def step(self, grad_scale: float = 1.0):
        if self.arena is not None:
            a = self.arena
            a.ctx.call("fml_sgd_step", a.values, a.grads, a.size, float(self.learningRate), float(grad_scale))
            return
        for p in self.parameters:
            if p.grad is not None:
                p.ctx.call("fml_sgd_step", p.value, p.grad, p.value.size, float(self.learningRate), float(grad_scale))


class Adam(Optimizer):
    """lib/optimizers/adam.dart:14-78: beta1 0.9, beta2 0.999, epsilon 1e-8, per-parameter m and v,
    step counter incremented before use (:46)."""

    def __init__(self, parameters, learningRate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, arena=None):
        super().__init__(parameters, learningRate, arena)
        self.beta1, self.beta2, self.epsilon, self._t = beta1, beta2, epsilon, 0
        if arena is not None:
            self._m, self._v = arena.ctx.zeros(arena.size), arena.ctx.zeros(arena.size)
        else:
            self._m = [p.ctx.zeros(*p.value.shape) for p in parameters]
            self._v = [p.ctx.zeros(*p.value.shape) for p in parameters]

    def step(self, grad_scale: float = 1.0):
        self._t += 1
        hp = (float(self.learningRate), float(self.beta1), float(self.beta2), float(self.epsilon), self._t, float(grad_scale))
        if self.arena is not None:
            a = self.arena
            a.ctx.call("fml_adam_step", a.values, a.grads, self._m, self._v, a.size, *hp)
            return
        for p, m, v in zip(self.parameters, self._m, self._v):
            if p.grad is not None:
                p.ctx.call("fml_adam_step", p.value, p.grad, m, v, p.value.size, *hp)
