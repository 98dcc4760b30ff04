"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import register_block
from .base import Block, FeedForward, Mixer, Norm, Prenormed, RunBinding, StepContext


@register_block("prenorm")
class PreNormBlock(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +x
    (crates/aien-inference-abi/src/weights.rs:290-365).  Each residual sum is carried as a
    pending ``delta`` and added inside the next norm kernel; or, where the norm and the parts
    around it allow (``Norm.sink``), the product that ends a branch adds it and the product that
    follows finishes the norm, and no norm kernel runs between them."""

    norm_slots = ("norm_in", "norm_post")
    chains_norm = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm_in: Norm, norm_post: Norm):
        self.mixer, self.feed_forward, self.norm_in, self.norm_post = mixer, feed_forward, norm_in, norm_post

    def parts(self):
        return {"norm_in": self.norm_in, "mixer": self.mixer, "norm_post": self.norm_post, "feed_forward": self.feed_forward}

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values())

    def first_norm(self):
        return self.norm_in

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, run: RunBinding, next_norm: Optional[Norm] = None):
        h = self.norm_in.forward(ctx, x, delta)
        if isinstance(h, Prenormed) and not self.mixer.takes_prenormed:
            h = h.materialise(ctx)
        sink = self.norm_post.sink(ctx, x) if self.mixer.feeds_residual else None
        a = self.mixer.forward(ctx, h, run, sink=sink) if sink is not None else self.mixer.forward(ctx, h, run)
        h2 = self.norm_post.forward(ctx, x, a)
        if isinstance(h2, Prenormed) and not self.feed_forward.takes_prenormed:
            h2 = h2.materialise(ctx)
        sink = next_norm.sink(ctx, x) if (next_norm is not None and self.feed_forward.feeds_residual) else None
        return self.feed_forward.forward(ctx, h2, sink=sink) if sink is not None else self.feed_forward.forward(ctx, h2)
