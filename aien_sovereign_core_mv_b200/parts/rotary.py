"""Rotary position encoding: frequency table, optional llama3 smoothing, per-step cos/sin."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_position
from .base import Position, StepContext


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict] = None, rotary_dim: Optional[int] = None):
    """inv_freq_i = theta^(-2i/d) in float64 (theta itself held as float32, as the reference
    does), optionally smoothed the llama3 way (crates/aien-abi-core/src/lib.rs:69-84, 106-114)."""
    d = rotary_dim or head_dim
    theta32 = float(torch.tensor(theta, dtype=torch.float32).item())
    inv = [1.0 / theta32 ** ((2 * i) / d) for i in range(d // 2)]
    if scaling:
        old = float(scaling["original_max_position_embeddings"])
        low_w = old / scaling["low_freq_factor"]
        high_w = old / scaling["high_freq_factor"]
        out = []
        for f in inv:
            wavelen = 2.0 * math.pi / f
            if wavelen < high_w:
                out.append(f)
            elif wavelen > low_w:
                out.append(f / scaling["factor"])
            else:
                smooth = (old / wavelen - scaling["low_freq_factor"]) / (scaling["high_freq_factor"] - scaling["low_freq_factor"])
                out.append((1.0 - smooth) * f / scaling["factor"] + smooth * f)
        inv = out
    return inv


@register_position("rotary")
class RotaryPosition(Position):
    """rotate_half pairing (i, i + d/2); angle = position * inv_freq in float64, cos and sin
    rounded to float32 (crates/aien-inference-abi/src/tensor.rs:150-188).  The table of a step
    is built once and shared by every layer that uses the same part."""

    def __init__(self, head_dim: int, theta: float, scaling: Optional[dict] = None, rotary_dim: Optional[int] = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim or head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self._inv_host = inverse_frequencies(self.head_dim, self.theta, self.scaling, self.rotary_dim)
        self._inv_dev: Optional[torch.Tensor] = None

    def step_workspace_bytes(self, max_tokens):
        return 2 * (max_tokens * (self.rotary_dim // 2) * 4 + 256)

    def rotary(self, ctx: StepContext):
        key = ("rotary", id(self))
        hit = ctx.shared.get(key)
        if hit is None:
            if self._inv_dev is None:
                self._inv_dev = torch.tensor(self._inv_host, dtype=torch.float64, device=ctx.positions.device)
            half = self.rotary_dim // 2
            cos = ctx.workspace.take_step((ctx.num_tokens, half), torch.float32)
            sin = ctx.workspace.take_step((ctx.num_tokens, half), torch.float32)
            K.rope_table(ctx.positions, self._inv_dev, cos, sin)
            hit = (cos, sin, self.rotary_dim)
            ctx.shared[key] = hit
        return hit


@register_position("none")
class NoPosition(Position):
    """Positions enter nowhere (a mixer with its own notion of order)."""

    def __init__(self, **_):
        pass

    def rotary(self, ctx):
        return None

    def apply(self, ctx, q, group, run):
        return None
