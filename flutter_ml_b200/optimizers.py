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

    def begin_step(self):
        """Advance the step counter once (adam.dart:46) before the slices of one step are updated with `step_slice`."""
        self._t += 1

    def step_slice(self, offset: int, n: int, lane: int = 0, zero_grad: bool = True, grad_scale: float = 1.0):
        """The update of arena elements [offset, offset + n) enqueued on copy lane `lane`, clearing that part of the
        gradient in the same pass: lets the update of layers whose gradients are final (and exchanged) run under the
        backward pass of the layers below them."""
        a = self.arena
        sl = lambda buf: buf.ptr + 4 * offset  # noqa: E731
        a.ctx.check(a.ctx.lib.fml_adam_step_on(a.ctx.h, lane, sl(a.values), sl(a.grads), sl(self._m), sl(self._v), n,
                                               float(self.learningRate), float(self.beta1), float(self.beta2), float(self.epsilon),
                                               self._t, float(grad_scale), 1 if zero_grad else 0))
        a.ctx.launches += 1


class _StatefulOptimizer(Optimizer):
    """Shared host side of the optimizers that run through `fml_optimizer_step`: up to three
    zero-initialised state buffers shaped like the parameters (one flat buffer each with an arena)."""

    KIND, N_STATE = 0, 1

    def __init__(self, parameters, learningRate, arena=None):
        super().__init__(parameters, learningRate, arena)
        self._t = 0
        if arena is not None:
            self._state = [arena.ctx.zeros(arena.size) for _ in range(self.N_STATE)]
        else:
            self._state = [[p.ctx.zeros(*p.value.shape) for p in parameters] for _ in range(self.N_STATE)]

    def _hyper(self):
        raise NotImplementedError

    def step(self):
        self._t += 1
        h = tuple(float(v) for v in self._hyper()) + (0.0,) * 4
        tail = (float(self.learningRate), h[0], h[1], h[2], h[3], self._t)
        if self.arena is not None:
            a = self.arena
            s = list(self._state) + [None] * (3 - self.N_STATE)
            a.ctx.call("fml_optimizer_step", self.KIND, a.values, a.grads, s[0], s[1], s[2], a.size, *tail)
            return
        for i, p in enumerate(self.parameters):
            if p.grad is None:
                continue
            s = [st[i] for st in self._state] + [None] * (3 - self.N_STATE)
            p.ctx.call("fml_optimizer_step", self.KIND, p.value, p.grad, s[0], s[1], s[2], p.value.size, *tail)


class SGDMomentum(_StatefulOptimizer):
    """v = momentum*v + lr*g; w -= v (lib/optimizers/sgdmomentum.dart:56-57)."""
    KIND, N_STATE = 1, 1

    def __init__(self, parameters, learningRate, momentum=0.9, arena=None):
        super().__init__(parameters, learningRate, arena)
        self.momentum = momentum

    def _hyper(self):
        return (self.momentum,)


class NAG(_StatefulOptimizer):
    """v = momentum*v + g; w -= lr*(g + momentum*v) (lib/optimizers/nag.dart:58-60)."""
    KIND, N_STATE = 2, 1

    def __init__(self, parameters, learningRate, momentum=0.9, arena=None):
        super().__init__(parameters, learningRate, arena)
        self.momentum = momentum

    def _hyper(self):
        return (self.momentum,)


class RMSprop(_StatefulOptimizer):
    """s = beta*s + (1-beta)*g^2; w -= lr*g/(sqrt(s)+eps) (lib/optimizers/rmsprop.dart:57-58)."""
    KIND, N_STATE = 3, 1

    def __init__(self, parameters, learningRate, beta=0.99, epsilon=1e-8, arena=None):   # defaults of rmsprop.dart
        super().__init__(parameters, learningRate, arena)
        self.beta, self.epsilon = beta, epsilon

    def _hyper(self):
        return (self.beta, self.epsilon)


class Adagrad(_StatefulOptimizer):
    """s += g^2; w -= lr*g/(sqrt(s)+eps) (lib/optimizers/adagrad.dart:54-55)."""
    KIND, N_STATE = 4, 1

    def __init__(self, parameters, learningRate, epsilon=1e-8, arena=None):
        super().__init__(parameters, learningRate, arena)
        self.epsilon = epsilon

    def _hyper(self):
        return (0.0, self.epsilon)


class AdamW(_StatefulOptimizer):
    """Adam update followed by the decoupled decay w -= lr*weightDecay*w (lib/optimizers/adamw.dart:82-89)."""
    KIND, N_STATE = 6, 2

    def __init__(self, parameters, learningRate, beta1=0.9, beta2=0.999, epsilon=1e-8, weightDecay=0.01, arena=None):
        super().__init__(parameters, learningRate, arena)
        self.beta1, self.beta2, self.epsilon, self.weightDecay = beta1, beta2, epsilon, weightDecay

    def _hyper(self):
        return (self.beta1, self.beta2, self.epsilon, self.weightDecay)


class AMSGrad(_StatefulOptimizer):
    """Adam with the running maximum of v in the denominator (lib/optimizers/amsgrad.dart:80-86)."""
    KIND, N_STATE = 7, 3

    def __init__(self, parameters, learningRate, beta1=0.9, beta2=0.999, epsilon=1e-8, arena=None):
        super().__init__(parameters, learningRate, arena)
        self.beta1, self.beta2, self.epsilon = beta1, beta2, epsilon

    def _hyper(self):
        return (self.beta1, self.beta2, self.epsilon)
