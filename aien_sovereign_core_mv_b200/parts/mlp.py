"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from .. import kernels as K
from ..registry import register_feed_forward
from .base import FeedForward, StepContext
from .linear import linear


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """y = (silu(h Wg^T) * (h Wu^T)) Wd^T, no bias (crates/aien-inference-abi/src/
    transformer_backend.rs:1322-1362, silu in src/backend.rs:572-579).  gate and up are one
    product over the stacked rows gate | up (src/resident.rs:284-288)."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def param_shapes(self):
        H, I = self.hidden_size, self.intermediate_size
        return {"gate_proj": ((I, H), "matrix"), "up_proj": ((I, H), "matrix"), "down_proj": ((H, I), "matrix")}

    def bind(self, tensors):
        g, u = tensors["gate_proj"], tensors["up_proj"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def workspace_bytes(self, max_tokens, itemsize):
        return max_tokens * (3 * self.intermediate_size + self.hidden_size) * itemsize + 1024

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        gu = linear(ctx, h, self.w_gate_up)
        act = ctx.workspace.take((ctx.num_tokens, self.intermediate_size), ctx.dtype)
        K.swiglu(gu, act)
        return linear(ctx, act, self.w_down)
