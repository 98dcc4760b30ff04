from .base import (Block, CacheNeed, Embedding, FeedForward, GroupView, Head, Mixer, Norm, Part, Position, RunBinding,
                   StepContext, StepLimits, Workspace, add_to_residual)
from . import norm, rotary, attention, mlp, block, ends  # noqa: F401  (registers the built-in parts)
from .linear import linear

__all__ = ["Block", "CacheNeed", "Embedding", "FeedForward", "GroupView", "Head", "Mixer", "Norm", "Part", "Position",
           "RunBinding", "StepContext", "StepLimits", "Workspace", "add_to_residual", "linear"]
