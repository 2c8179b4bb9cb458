"""Layer arrangement, embedding and output head.

Pre-norm block with two residual sums (src/quanta/minimax/model.py:70-73):
``h = h + mixer(norm_1(h)); h = h + feed_forward(norm_2(h))``.  The sums are taken in float32 inside
the norm kernels: a part's output stays "pending" until the next norm reads the row.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Block, Embedding, Head, TensorSpec, make, register


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


@register("embedding", "token_table")
class TokenTable(Embedding):
    """``h = table[ids]`` into the float32 residual stream (src/quanta/minimax/model.py:91)."""

    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str):
        self.V, self.H, self.weight_name = int(vocab_size), int(hidden_size), weight_name
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.V, self.H))]

    def load(self, fetch):
        self.table = fetch(self.weight_name)

    def forward(self, ids, ctx):
        h = torch.empty((ids.numel(), self.H), dtype=torch.float32, device=ids.device)
        kernels.embedding(h, self.table, ids, ctx.status)
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
