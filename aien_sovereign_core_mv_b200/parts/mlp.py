"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from .. import kernels as K
from ..registry import register_feed_forward
from typing import Optional

from .base import FeedForward, Prenormed, ResidualSink, StepContext
from .linear import linear, linear_into_residual, linear_prenormed, _FORCE


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

    GROUP = 8      # gate and up rows interleaved in runs of 8: one decode-kernel tile holds both

    def bind(self, tensors):
        g, u = tensors["gate_proj"], tensors["up_proj"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        I, H = self.intermediate_size, self.hidden_size
        self.group = self.GROUP if (g.dtype == torch.bfloat16 and I % self.GROUP == 0) else 0
        if self.group:
            n = I // self.group
            self.w_gate_up = torch.stack([g.view(n, self.group, H), u.view(n, self.group, H)], dim=1).reshape(2 * I, H).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def workspace_bytes(self, lim):
        return lim.max_tokens * (3 * self.intermediate_size + self.hidden_size) * lim.itemsize + 4096 \
            + 8 * K.GEMV_MAX_ROWS * self.hidden_size * 4 + K.PARTIALS_MAX_BYTES + K.FUSED_NORM_SCRATCH_BYTES(self.hidden_size)

    takes_prenormed = True
    feeds_residual = True

    def forward(self, ctx: StepContext, h, sink: Optional[ResidualSink] = None):
        if isinstance(h, Prenormed):
            act = linear_prenormed(ctx, h, self.w_gate_up, epilogue=1) if self.group == 8 else None
            if act is not None:
                return linear_into_residual(ctx, act, self.w_down, sink) or linear(ctx, act, self.w_down, may_defer_sum=True)
            h = h.materialise(ctx)
        act = ctx.workspace.take((ctx.num_tokens, self.intermediate_size), ctx.dtype)
        if self.group == 8 and h.shape[0] <= K.GEMV_ROUTE_ROWS and K.gemv_supports(h, self.w_gate_up, act):
            K.gemv(h, self.w_gate_up, act, epilogue=1)          # silu(gate)*up inside the product
        elif self.group == 8 and K.gemm_tc_supports(h, self.w_gate_up, act) and not _FORCE:
            K.gemm_tc(h, self.w_gate_up, act, epilogue=1)       # the same, in the tensor-core epilogue
        else:
            gu = linear(ctx, h, self.w_gate_up)
            K.swiglu(gu, act, self.group)
        return linear_into_residual(ctx, act, self.w_down, sink) or linear(ctx, act, self.w_down, may_defer_sum=True)
