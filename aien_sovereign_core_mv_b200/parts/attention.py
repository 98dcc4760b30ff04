"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_mixer
from .base import CacheNeed, Mixer, Position, Prenormed, ResidualSink, RunBinding, StepContext
from .linear import linear, linear_into_residual, linear_prenormed


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    """q/k/v projection (one product over the stacked rows q|k|v), optional per-head RMSNorm of
    q and k before rotation, rotation, write of k and v into the token's cache slot, causal
    attention over the request's pages (optionally only the last ``window`` keys), output
    projection.  Formulas: crates/aien-inference-abi/src/transformer_backend.rs:1229-1319 and
    src/backend.rs:311-379; the stacked q|k|v rows follow src/resident.rs:284-288.

    A run that does not write its cache (``run.writes == False``) projects q only and attends
    over the planes another run filled."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: Position,
                 qk_norm: bool = False, qk_norm_eps: float = 1e-6, window: int = 0, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take even sizes up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.position = position
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_dim, self.kv_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---- tensors
    def param_shapes(self):
        H = self.hidden_size
        shapes = {
            "q_proj": ((self.q_dim, H), "matrix"), "k_proj": ((self.kv_dim, H), "matrix"),
            "v_proj": ((self.kv_dim, H), "matrix"), "o_proj": ((H, self.q_dim), "matrix"),
        }
        if self.qk_norm:
            shapes["q_norm"] = ((self.head_dim,), "norm")
            shapes["k_norm"] = ((self.head_dim,), "norm")
        return shapes

    def bind(self, tensors):
        q, k, v = tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()       # rows q | k | v
        self.w_o = tensors["o_proj"].contiguous()
        if self.qk_norm:
            qn, kn = tensors["q_norm"], tensors["k_norm"]
            if qn.dtype != kn.dtype:
                qn, kn = qn.float(), kn.float()
            self.q_norm_w, self.k_norm_w = qn.contiguous(), kn.contiguous()

    def cache_need(self):
        return CacheNeed.keys_and_values("window" if self.window > 0 else "full", self.window, self.num_kv_heads, self.head_dim)

    def workspace_bytes(self, lim):
        return lim.max_tokens * (2 * self.q_dim + 2 * self.kv_dim + self.q_dim + self.hidden_size) * lim.itemsize + 4096 \
            + 8 * K.GEMV_MAX_ROWS * (self.q_dim + 2 * self.kv_dim + self.hidden_size) * 4 + 2 * K.PARTIALS_MAX_BYTES \
            + K.attention_workspace_bytes(lim, self.num_heads, self.head_dim) + K.FUSED_NORM_SCRATCH_BYTES(self.hidden_size)

    # ---- one step
    takes_prenormed = True
    feeds_residual = True

    def _project(self, ctx: StepContext, h, w: torch.Tensor) -> torch.Tensor:
        if isinstance(h, Prenormed):
            y = linear_prenormed(ctx, h, w)
            if y is not None:
                return y
            h = h.materialise(ctx)
        return linear(ctx, h, w, may_defer_sum=True)

    def forward(self, ctx: StepContext, h, run: RunBinding, sink: Optional[ResidualSink] = None):
        T = ctx.num_tokens
        group = ctx.groups[run.group]
        k_cache, v_cache = group.storage["k"][run.slot], group.storage["v"][run.slot]     # [tokens, nkv, hd] each
        if run.writes:
            qkv = self._project(ctx, h, self.w_qkv)
            q, k, v = qkv[..., :self.q_dim], qkv[..., self.q_dim:self.q_dim + self.kv_dim], qkv[..., self.q_dim + self.kv_dim:]
        else:
            q = self._project(ctx, h, self.w_qkv[:self.q_dim])
            k = v = None
        rot = self.position.rotary(ctx)
        cos, sin, rdim = rot if rot is not None else (None, None, 0)
        if (K._FORCE_ATTN == "fused" and ctx.decode_only and run.writes and q.dim() == 2 and rot is not None
                and K.decode_attention_supports(q, k_cache, self.num_heads, self.num_kv_heads, self.head_dim)):
            # One launch: q/k norm, rotation, cache write and attention.  Opt-in (AIEN_B200_ATTENTION=fused):
            # measured on the Qwen3-8B shape it equals the two launches at batch 1 and loses at batch 8
            # and 64, where every chunk's CTA repeats the q work.
            out = ctx.workspace.take((T, self.q_dim), ctx.dtype)
            K.paged_attention_decode_fused(ctx, q, k, v, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, cos, sin, rdim, group,
                                           k_cache, v_cache, out, self.num_heads, self.num_kv_heads, self.head_dim,
                                           self.window, self.scale)
            return linear(ctx, out, self.w_o, may_defer_sum=True)
        q_out = ctx.workspace.take((T, self.q_dim), ctx.dtype) if q.dim() == 3 else q
        K.qk_norm_rope_kv_write(q, k, v, self.head_dim, self.q_norm_w, self.k_norm_w if k is not None else None,
                                self.qk_norm_eps, cos, sin, rdim,
                                group.slot_map if k is not None else None,
                                k_cache if k is not None else None, v_cache if k is not None else None, q_out=q_out)
        if rot is None:
            self.position.apply(ctx, q_out, group, run)
        out = ctx.workspace.take((T, self.q_dim), ctx.dtype)
        K.paged_attention(ctx, q_out, k_cache, v_cache, group, out, self.num_heads, self.num_kv_heads, self.head_dim,
                          self.window, self.scale)
        return linear_into_residual(ctx, out, self.w_o, sink) or linear(ctx, out, self.w_o, may_defer_sum=True)
