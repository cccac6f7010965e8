"""SNetwork: the reference's model container (lib/nets/snet.dart:34-157)."""
from __future__ import annotations

import time
from typing import List

from . import tensor as T
from .layers import Layer
from .tensor import Tensor


class SNetwork(Layer):
    name = "snetwork"

    def __init__(self, layers: List[Layer]):
        super().__init__()
        self.layers = layers
        self.optimizer = None

    @property
    def parameters(self):
        return [p for layer in self.layers for p in layer.parameters]

    def predict(self, x: Tensor) -> Tensor:
        return self.forward(x)

    def forward(self, x: Tensor) -> Tensor:
        """snet.dart:51-57."""
        for layer in self.layers:
            x = layer.call(x)
        return x

    def call(self, x):
        return self.forward(x)

    def compile(self, configuredOptimizer):
        self.optimizer = configuredOptimizer

    def fit(self, inputs: List[Tensor], targets: List[Tensor], epochs: int, loss=T.mseMatrix, verbose: bool = False):
        """One optimizer step per sample: forward, loss, backward, step, zeroGrad
        (snet.dart:71-85).  Returns the average loss of each epoch."""
        assert self.optimizer is not None, "call compile(optimizer) first"
        t0 = time.perf_counter()
        history = []
        for epoch in range(epochs):
            total = 0.0
            for x, y in zip(inputs, targets):
                out = self.forward(x)
                l = loss(out, y)
                l.backward()
                self.optimizer.step()
                self.optimizer.zeroGrad()
                total += float(l.numpy()[0])
            history.append(total / max(1, len(inputs)))
            if verbose:
                print(f"epoch {epoch + 1}/{epochs} avg loss {history[-1]:.6f}")
        self.last_fit_seconds = time.perf_counter() - t0
        return history

    def fitBatched(self, inputs, targets, batch_size: int, epochs: int, loss=T.mseMatrix, shuffle_seed=None,
                   drop_last: bool = False, verbose: bool = False):
        """fit() over HOST arrays, one optimizer step per batch of rows (the step sequence of snet.dart:74-85 with
        a batch matrix in place of one sample).  `inputs` [n x features] and `targets` ([n x outputs] floats, or
        [n] integer labels for a loss that takes labels) stay in host memory; a BatchFeeder uploads batch s+1 on
        a copy lane while batch s trains, the per-batch losses are summed on the device and read back once per
        epoch, so no step waits for the host.  `shuffle_seed` draws one permutation per epoch from
        numpy's default_rng(seed + epoch); None keeps the given order.  Returns the average batch loss per epoch."""
        import numpy as np
        from .feeder import BatchFeeder
        assert self.optimizer is not None, "call compile(optimizer) first"
        ctx = self.parameters[0].ctx
        feeder = BatchFeeder(ctx, [np.asarray(inputs), np.asarray(targets)], batch_size, drop_last=drop_last)
        self.feeder = feeder
        loss_sum = ctx.zeros(1)
        t0 = time.perf_counter()
        history = []
        for epoch in range(epochs):
            order = None
            if shuffle_seed is not None:
                order = np.random.default_rng(shuffle_seed + epoch).permutation(feeder.n)
            ctx.zero(loss_sum)
            steps = 0
            for x, y in feeder.batches(order):
                out = self.forward(Tensor(x))
                l = loss(out, Tensor(y) if y.dtype == np.float32 else y)
                l.backward()
                self.optimizer.step()
                self.optimizer.zeroGrad()
                ctx.call("fml_axpy", 1.0, l.value, loss_sum, 1)
                steps += 1
            history.append(float(loss_sum.numpy()[0]) / max(1, steps))   # the one host read of the epoch
            if verbose:
                print(f"epoch {epoch + 1}/{epochs} avg loss {history[-1]:.6f}")
        self.last_fit_seconds = time.perf_counter() - t0
        return history

    def evaluate(self, inputs: List[Tensor], targets: List[Tensor]) -> float:
        """Fraction of samples whose rounded prediction equals the target (snet.dart:144-156)."""
        import numpy as np
        ok = 0
        for x, y in zip(inputs, targets):
            if np.array_equal(np.round(self.forward(x).numpy()), np.round(y.numpy())):
                ok += 1
        return ok / max(1, len(inputs))
