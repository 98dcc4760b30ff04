"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import register_block
from .base import Block, FeedForward, Mixer, Norm, RunBinding, StepContext


@register_block("prenorm")
class PreNormBlock(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +x
    (crates/aien-inference-abi/src/weights.rs:290-365).  Each residual sum is carried as a
    pending ``delta`` and added inside the next norm kernel."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm_in: Norm, norm_post: Norm):
        self.mixer, self.feed_forward, self.norm_in, self.norm_post = mixer, feed_forward, norm_in, norm_post

    def parts(self):
        return {"norm_in": self.norm_in, "mixer": self.mixer, "norm_post": self.norm_post, "feed_forward": self.feed_forward}

    def workspace_bytes(self, lim):
        return sum(p.workspace_bytes(lim) for p in self.parts().values())

    def forward(self, ctx: StepContext, x: torch.Tensor, delta: Optional[torch.Tensor], run: RunBinding) -> torch.Tensor:
        h = self.norm_in.forward(ctx, x, delta)
        a = self.mixer.forward(ctx, h, run)
        h2 = self.norm_post.forward(ctx, x, a)
        return self.feed_forward.forward(ctx, h2)
