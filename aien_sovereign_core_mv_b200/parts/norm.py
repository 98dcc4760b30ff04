"""RMSNorm with the residual sum fused in front of it."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_norm
from .base import Norm, Prenormed, ResidualSink, StepContext

# AIEN_B200_FUSED_NORM=0 keeps every norm in its own kernel
_FUSE = __import__("os").environ.get("AIEN_B200_FUSED_NORM", "1").strip() not in ("0", "off", "no")


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """h = x * (1/sqrt(mean(x^2) + eps)) * w over the last axis
    (crates/aien-inference-abi/src/tensor.rs:94-110).  The sum of squares and the scale are
    float32; x is the float32 residual stream and is updated in place when ``delta`` is given."""

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {"weight": ((self.size,), "norm")}

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def workspace_bytes(self, lim):
        return lim.max_tokens * self.size * lim.itemsize + 256

    def sink(self, ctx: StepContext, x: torch.Tensor) -> Optional[ResidualSink]:
        if not _FUSE or not K.small_step_products_fuse(ctx.dtype, ctx.num_tokens):
            return None
        return ResidualSink(x, self, self.weight, self.eps)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta):
        if isinstance(delta, Prenormed):
            if delta.norm is self:
                return delta                      # the sum is in x already; the consumer finishes the norm
            delta = None                          # made for another norm: x is up to date, norm it here
        out = ctx.workspace.take(tuple(x.shape), ctx.dtype)
        K.add_rmsnorm(x, delta, self.weight, self.eps, out)
        return out
