from .base import (Block, CacheNeed, FeedForward, GroupView, Mixer, Norm, Part, Position, RunBinding,
                   StepContext, StepLimits, Workspace)
from . import norm, rotary, attention, mlp, block  # noqa: F401  (registers the built-in parts)
from .linear import linear

__all__ = ["Block", "CacheNeed", "FeedForward", "GroupView", "Mixer", "Norm", "Part", "Position",
           "RunBinding", "StepContext", "StepLimits", "Workspace", "linear"]
