"""Layer arrangement, embedding and output head.

Pre-norm block with two residual sums (src/quanta/minimax/model.py:70-73):
``h = h + mixer(norm_1(h)); h = h + feed_forward(norm_2(h))``.  The sums are taken in float32 inside
the norm kernels: a part's output stays "pending" until the next norm reads the row.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Block, Embedding, Head, NormedPending, TensorSpec, make, register


@register("block", "pre_norm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, hidden_size: int, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.hidden = int(hidden_size)
        self.mixer = make("mixer", mixer)
        self.feed_forward = make("feed_forward", feed_forward)
        self.mixer_norm = make("norm", mixer_norm)
        self.feed_forward_norm = make("norm", feed_forward_norm)

    def children(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, h, pending, ctx, cache, state):
        x = empty_rows(h.shape[0], self.hidden, dtype=ctx.dtype, device=h.device)
        self.mixer_norm.forward(h, pending, x)
        a = self.mixer.forward(x, ctx, cache, state)
        x2 = empty_rows(h.shape[0], self.hidden, dtype=ctx.dtype, device=h.device)
        self.feed_forward_norm.forward(h, a, x2)
        return self.feed_forward.forward(x2, ctx)


@register("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after each sublayer: ``h += post_1(mixer(conv(pre_1(h))))`` and, where the
    layer has a feed-forward, ``h += post_2(feed_forward(pre_2(h)))``.  ``conv`` (optional) is a short
    convolution over time on the mixer's input; its last inputs are part of the layer's per-request state.
    Both sums are float32 and happen inside the next pre-norm (or the head's norm), which also applies the
    post-norm to the sublayer's float32 output: a contribution is never rounded to the activation dtype."""

    graph_safe = True

    def __init__(self, hidden_size: int, mixer, mixer_norm, mixer_post_norm, feed_forward=None,
                 feed_forward_norm=None, feed_forward_post_norm=None, conv=None):
        self.hidden = int(hidden_size)
        self.mixer = make("mixer", mixer)
        self.mixer_norm = make("norm", mixer_norm)
        self.mixer_post_norm = make("norm", mixer_post_norm)
        self.conv = make("time_conv", conv) if conv is not None else None
        self.feed_forward = make("feed_forward", feed_forward) if feed_forward is not None else None
        self.feed_forward_norm = self.feed_forward_post_norm = None
        if self.feed_forward is not None:
            self.feed_forward_norm = make("norm", feed_forward_norm)
            self.feed_forward_post_norm = make("norm", feed_forward_post_norm)

    def children(self):
        parts = [self.mixer_norm, self.conv, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                 self.feed_forward, self.feed_forward_post_norm]
        return [p for p in parts if p is not None]

    def state_spec(self):
        spec = dict(self.mixer.state_spec())
        if self.conv is not None:
            for name, need in self.conv.state_spec().items():
                if name in spec:
                    raise ValueError(f"the mixer and the convolution both keep a state named {name!r}")
                spec[name] = need
        return spec

    def forward(self, h, pending, ctx, cache, state):
        T = h.shape[0]
        x = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device)
        if self.conv is None:
            self.mixer_norm.forward(h, pending, x)
        else:
            normed = torch.empty((T, self.hidden), dtype=torch.float32, device=h.device)
            self.mixer_norm.forward(h, pending, normed)
            self.conv.forward(normed, ctx, state, x)
        # a sublayer's output stays pending together with its post-norm: the next pre-norm (or the head's norm)
        # norms it, adds it to the stream and norms the sum in one launch
        d = NormedPending(self.mixer.forward(x, ctx, cache, state), self.mixer_post_norm)
        if self.feed_forward is None:
            return d
        x2 = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device)
        self.feed_forward_norm.forward(h, d, x2)
        return NormedPending(self.feed_forward.forward(x2, ctx), self.feed_forward_post_norm)


@register("embedding", "token_table")
class TokenTable(Embedding):
    """``h = table[ids] * scale`` into the float32 residual stream (src/quanta/minimax/model.py:91; the
    reference has no scale)."""

    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, scale: float = 1.0):
        self.V, self.H, self.weight_name, self.scale = int(vocab_size), int(hidden_size), weight_name, float(scale)
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.V, self.H))]

    def load(self, fetch):
        self.table = fetch(self.weight_name)

    def forward(self, ids, ctx):
        h = torch.empty((ids.numel(), self.H), dtype=torch.float32, device=ids.device)
        kernels.embedding(h, self.table, ids, ctx.status, self.scale)
        return h


@register("head", "linear")
class LinearHead(Head):
    """Final norm on the wanted rows, then ``logits = x @ head.T`` in float32
    (src/quanta/minimax/runtime.py:95-98).  ``tied_to`` names the embedding table to reuse (a tensor that
    two parts ask for by the same name is loaded once and shared)."""

    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, norm, weight_name: str | None, tied_to: str | None):
        self.V, self.H = int(vocab_size), int(hidden_size)
        self.norm = make("norm", norm)
        self.weight_name, self.tied_to = weight_name, tied_to
        self.weight = None

    def children(self):
        return [self.norm]

    def tensor_specs(self):
        return [TensorSpec(self.tied_to if self.tied_to else self.weight_name, (self.V, self.H))]

    def load(self, fetch):
        self.weight = fetch(self.tied_to if self.tied_to else self.weight_name)

    def forward(self, h, pending, rows, ctx):
        n = rows.numel()
        x = empty_rows(n, self.H, dtype=ctx.dtype, device=h.device)
        self.norm.forward(h, pending, x, rows=rows, store_h=False)
        return linear(x, self.weight, out_dtype=torch.float32)
