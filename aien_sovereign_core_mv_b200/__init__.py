"""A small, whole inference engine for the dense Llama / Qwen3 decoder on one B200 (sm_100a).

Public surface: :class:`Engine` (model + cache + step), :class:`EngineConfig`,
``generate`` (Python entry point), the registries for architectures and parts, and the weight
tools (random model folders, checkpoint errors).
"""
from .config import ConfigError, DenseDecoderConfig, EngineConfig, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (register_architecture, register_block, register_embedding, register_feed_forward, register_head,
                       register_mixer, register_norm, register_position)
from .weights import WeightError, SafetensorsError
from . import models as _models  # noqa: F401  (registers the built-in architectures and parts)
from .models.loading import write_random_model, model_spec_for
from .engine import Engine, StepEntry

__all__ = [
    "ConfigError", "DenseDecoderConfig", "EngineConfig", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry",
    "register_architecture", "register_block", "register_embedding", "register_feed_forward", "register_head",
    "register_mixer", "register_norm", "register_position", "WeightError", "SafetensorsError", "write_random_model", "model_spec_for",
    "Engine", "StepEntry",
]
__version__ = "0.1.0"
