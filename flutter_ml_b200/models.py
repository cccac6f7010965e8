"""The benchmark configurations assembled from the reference-shaped layers.

    config 1  MLP 784-128-64-10, ReLU, softmax cross-entropy, SGD        -> `MLP`
    config 3  one post-LN encoder block, forward + backward               -> `encoder_block_fwd_bwd`
    config 5  Embedding -> +PE -> N blocks -> vocab head, Adam, data parallel -> `TransformerLM`

Weights are supplied by the caller (numpy, float32) so that tests can hand the identical values to
a CPU checker; `init_*` build them from the seeded generator the way the configurations state.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

from . import synth
from . import tensor as T
from .layers import DenseLayerMatrix, EmbeddingLayer, MultiHeadAttention, TransformerEncoderBlock
from .optimizers import SGD, Adam, ParameterArena
from .tensor import Tensor


# ----------------------------------------------------------------------------------- config 1
def init_mlp(seed: int = 0, sizes=(784, 128, 64, 10)) -> List[np.ndarray]:
    """Xavier-uniform weights [in x out] and zero biases, in order [W1,b1,W2,b2,W3,b3]."""
    out = []
    for i, (a, b) in enumerate(zip(sizes[:-1], sizes[1:])):
        out += [synth.xavier_uniform(seed, 10 + i, a, b), np.zeros(b, dtype=np.float32)]
    return out


class MLP:
    """DenseLayerMatrix(128,ReLU) -> DenseLayerMatrix(64,ReLU) -> DenseLayerMatrix(10) trained with softmax
    cross-entropy (mean over the batch) and SGD, one step = forward, loss, backward, step, zeroGrad
    (lib/nets/snet.dart:74-85)."""

    def __init__(self, ctx, params: List[np.ndarray], lr: float = 0.01, precision: int = -1):
        self.ctx = ctx
        n = len(params) // 2
        self.layers = [DenseLayerMatrix(params[2 * i].shape[1], "relu" if i < n - 1 else None, weights=params[2 * i],
                                        bias=params[2 * i + 1], precision=precision) for i in range(n)]
        x0 = Tensor(ctx.zeros(1, params[0].shape[0]), ctx)
        h = x0
        for layer in self.layers:
            h = layer(h)
        self.parameters = [p for layer in self.layers for p in layer.parameters]
        self.arena = ParameterArena(ctx, self.parameters)
        self.optimizer = SGD(self.parameters, lr, self.arena)

    def forward(self, x: Tensor) -> Tensor:
        for layer in self.layers:
            x = layer(x)
        return x

    def train_step(self, X, labels, keep=False):
        """X: DeviceArray [B x in], labels: int32 DeviceArray [B].  Returns the loss tensor (device)."""
        logits = self.forward(Tensor(X, self.ctx))
        logits_copy = None
        if keep:
            logits_copy = self.ctx.empty(*logits.shape)
            self.ctx.copy(logits_copy, logits.value)
        loss = T.softmaxCrossEntropy(logits, labels, 1.0 / X.shape[0])
        loss.backward()
        grads = self.arena.grads.numpy().copy() if keep else None
        self.optimizer.step()
        self.optimizer.zeroGrad()
        return loss, logits_copy, grads


    def record_step(self, X, labels):
        """Record one training step on (X, labels) as a CUDA graph.  The step is launch-bound (~15 kernels of a few
        microseconds each); replaying the graph issues them with one call.  X and labels are read from the
        same device buffers at every replay (refill them in place); the loss lands in `self.loss`."""
        import gc
        ctx = self.ctx
        self.train_step(X, labels)          # eager once: sizes the scratch arena, fills the tensor-map cache
        self.loss = ctx.zeros(1)
        gc.collect()
        n0 = ctx.launches
        ctx.graph_begin()
        try:
            loss, _, _ = self.train_step(X, labels)
            ctx.copy(self.loss, loss.value)
            del loss
            gc.collect()                    # every buffer allocated while recording is freed while recording
        finally:
            self._graph = ctx.graph_end()
        self._graph_launches = ctx.launches - n0
        return self._graph

    def replay_step(self):
        self.ctx.graph_launch(self._graph, launches=self._graph_launches)


# ----------------------------------------------------------------------------------- config 3
def init_block(seed: int, d_model: int, heads: int, dff: int, std: float = 0.02, tid: int = 0) -> Dict:
    """Encoder-block weights N(0, std), LayerNorm gamma 1 / beta 0, biases 0."""
    dk = d_model // heads
    n = lambda i, shape: synth.normal(seed, tid + i, shape, std)  # noqa: E731
    return {"heads": [tuple(n(3 * h + j, (d_model, dk)) for j in range(3)) for h in range(heads)],
            "Wo": n(1000, (d_model, d_model)),
            "g1": np.ones(d_model, np.float32), "be1": np.zeros(d_model, np.float32),
            "W1": n(1001, (d_model, dff)), "b1": np.zeros(dff, np.float32),
            "W2": n(1002, (dff, d_model)), "b2": np.zeros(d_model, np.float32),
            "g2": np.ones(d_model, np.float32), "be2": np.zeros(d_model, np.float32)}


def block_grads_in_reference_order(block: TransformerEncoderBlock, heads: int):
    """Gradients as numpy arrays in the order per-head (Wq,Wk,Wv)..., Wo, g1, be1, W1, b1, W2, b2, g2, be2."""
    gq = block.attention.Wqkv.grad.numpy()
    out = []
    for h in MultiHeadAttention.unpack_heads(gq, heads):
        out += list(h)
    for p in (block.attention.Wo, block.norm1.gamma, block.norm1.beta, block.ffn1.weights, block.ffn1.biases,
              block.ffn2.weights, block.ffn2.biases, block.norm2.gamma, block.norm2.beta):
        out.append(p.grad.numpy())
    return out


def encoder_block_fwd_bwd(ctx, x: np.ndarray, params: Dict, target: np.ndarray, heads: int, causal: bool = True,
                          precision: int = -1):
    """x, target: [n_seq, seq_len, d].  Loss = sum over sequences of mseMatrix(y_s, target_s).
    Returns (y, loss, dx, grads in reference order)."""
    n_seq, S, d = x.shape
    dff = params["W1"].shape[1]
    block = TransformerEncoderBlock(d, heads, dff, seq_len=S, causal=causal, params=params, precision=precision)
    xt = Tensor(ctx.upload(x.reshape(n_seq * S, d)), ctx)
    y = block(xt)
    # sum over sequences of per-sequence means = n_seq * mean over everything
    loss = T.mseMatrix(y, Tensor(ctx.upload(target.reshape(n_seq * S, d)), ctx), weight=float(n_seq))
    loss.backward()
    return (y.numpy().reshape(n_seq, S, d), float(loss.numpy()[0]), xt.grad.numpy().reshape(n_seq, S, d),
            block_grads_in_reference_order(block, heads))


# ----------------------------------------------------------------------------------- config 5
def init_lm(seed: int, vocab: int, d_model: int, heads: int, dff: int, layers: int, std: float = 0.02) -> Dict:
    return {"emb": synth.normal(seed, 1, (vocab, d_model), std),
            "blocks": [init_block(seed, d_model, heads, dff, std, tid=10000 * (i + 1)) for i in range(layers)],
            "Whead": synth.normal(seed, 2, (d_model, vocab), std), "bhead": np.zeros(vocab, np.float32)}


class TransformerLM:
    """EmbeddingLayer -> PositionalEncoding -> N x TransformerEncoderBlock (causal) -> DenseLayerMatrix(vocab)
    -> softmax cross-entropy over all tokens, Adam.  One data-parallel rank: the loss is normalised by
    the GLOBAL token count, gradients are summed across ranks by one all-reduce over the flat arena."""

    def __init__(self, ctx, params: Dict, seq_len: int, heads: int, lr: float = 1e-3, causal: bool = True,
                 precision: int = -1, rank: int = 0, world: int = 1):
        self.ctx, self.S, self.heads, self.rank, self.world = ctx, seq_len, heads, rank, world
        vocab, d = params["emb"].shape
        self.vocab, self.d = vocab, d
        self.embedding = EmbeddingLayer(vocab, d, positional_max_len=seq_len, table=params["emb"])
        self.embedding.build_on(ctx)
        self.blocks = [TransformerEncoderBlock(d, heads, b["W1"].shape[1], seq_len=seq_len, causal=causal, params=b,
                                               precision=precision) for b in params["blocks"]]
        self.head = DenseLayerMatrix(vocab, None, weights=params["Whead"], bias=params["bhead"], precision=precision)
        probe = Tensor(ctx.zeros(seq_len, d), ctx)
        h = probe
        for blk in self.blocks:
            h = blk(h)
        self.head(h)
        self.parameters = self.embedding.parameters + [p for b in self.blocks for p in b.parameters] + self.head.parameters
        self.arena = ParameterArena(ctx, self.parameters)
        self.optimizer = Adam(self.parameters, lr, arena=self.arena)
        del probe, h

    def _slice(self, first_param: int, n_params: int):
        """(offset, length) in the arena of `n_params` consecutive parameters."""
        offs = self.arena.offsets
        end = offs[first_param + n_params] if first_param + n_params < len(offs) else self.arena.size
        return offs[first_param], end - offs[first_param]

    def _exchange(self, off: int, n: int, update: bool = False):
        """Sum one finished slice of the gradient arena across ranks on the communication lane, after
        everything queued so far on the main stream; with `update`, apply Adam to that slice (and clear its
        gradient) on the same lane right behind the exchange."""
        c = self.ctx
        c.check(c.lib.fml_event_record_on(c.h, 50, -1))
        c.check(c.lib.fml_wait_event(c.h, 0, 50))
        if self.world > 1:
            c.check(c.lib.fml_dp_allreduce_sum_on(c.h, 0, self.arena.grads.ptr + 4 * off, n))
        if update:
            self.optimizer.step_slice(off, n, lane=0, zero_grad=True)

    def forward_backward(self, ids, labels, n_global_tokens: int, keep_logits: bool = False, overlap_exchange: bool = False,
                         fused_update: bool = False):
        """ids, labels: int32 DeviceArrays [n_seq * seq_len] of this rank's shard.  With
        `overlap_exchange` the all-reduce of each finished slice of the gradient arena (head, then the
        blocks from last to first, then the embedding) runs on a side stream under the rest of backward;
        with `fused_update` the Adam update of each slice follows its exchange on that stream, so that only the
        embedding table's exchange and update remain after the last backward kernel."""
        ctx = self.ctx
        h = self.embedding(ids)
        inputs = []
        for blk in self.blocks:
            inputs.append(h)
            h = blk(h)
        inputs.append(h)
        logits = self.head(h)
        before = None
        if fused_update or (overlap_exchange and self.world > 1):
            per_block = len(self.blocks[0].parameters)
            L = len(self.blocks)
            ex = lambda first, count: self._exchange(*self._slice(first, count), update=fused_update)  # noqa: E731
            before = {id(inputs[L]): (lambda: ex(1 + L * per_block, 2))}
            for i in range(L - 1, -1, -1):
                before[id(inputs[i])] = (lambda i=i: ex(1 + i * per_block, per_block))
        kept = None
        if keep_logits:
            kept = ctx.empty(*logits.shape)
            ctx.copy(kept, logits.value)
        loss = T.softmaxCrossEntropy(logits, labels, 1.0 / n_global_tokens, bias_grad=True)
        loss.backward(before=before)
        if before:
            self._exchange(*self._slice(0, 1), update=fused_update)   # the embedding table's gradient, last
            c = self.ctx
            c.check(c.lib.fml_event_record_on(c.h, 51, 0))  # main stream continues once the lane is done
            c.check(c.lib.fml_wait_event(c.h, -1, 51))
        return loss, kept

    def train_step(self, ids, labels, n_global_tokens: int, overlap_exchange: bool = True):
        """One step: forward, loss, backward, exchange, Adam, zeroGrad (lib/nets/snet.dart:74-85).  With
        `overlap_exchange` (the default) the exchange and the update run slice by slice on the side stream."""
        if overlap_exchange:
            self.optimizer.begin_step()
            loss, _ = self.forward_backward(ids, labels, n_global_tokens, overlap_exchange=True, fused_update=True)
            return loss
        loss, _ = self.forward_backward(ids, labels, n_global_tokens)
        if self.world > 1:
            self.ctx.call("fml_dp_allreduce_sum", self.arena.grads, self.arena.size)
        self.optimizer.step()
        self.optimizer.zeroGrad()
        return loss

    def check_values(self):
        """(gradient-independent) figures that every rank count must reproduce after a step: the L2 norm and a
        position-weighted checksum of the parameter arena, computed on the host in float64."""
        w = self.arena.values.numpy().astype(np.float64)
        return {"param_norm": float(np.sqrt(np.sum(w * w))), "param_checksum": float(np.sum(w * ((np.arange(w.size) % 251) + 1.0)))}

    def grads_in_reference_order(self):
        out = [self.embedding.embeddings.grad.numpy()]
        for b in self.blocks:
            out += block_grads_in_reference_order(b, self.heads)
        return out + [self.head.weights.grad.numpy(), self.head.biases.grad.numpy()]
