"""From a model folder (or a configuration and a seed) to a decoder with its weights bound."""
from __future__ import annotations

from typing import Mapping, Optional, Tuple

from ..config.model_config import ConfigError, read_config_json, read_generation_config
from ..config.spec import ModelSpec
from ..registry import get_architecture
from ..weights.loader import iter_checkpoint
from ..weights.random_init import random_tensors, write_model_folder
from .decoder import Decoder


def model_spec_for(raw_config: Mapping, generation_config: Optional[Mapping] = None, strict: bool = False):
    """(typed config, ModelSpec) for a parsed config.json, through the architecture registry."""
    archs = raw_config.get("architectures") if isinstance(raw_config, Mapping) else None
    if not isinstance(archs, (list, tuple)) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"config.json: architectures must name exactly one architecture, got {archs!r}")
    try:
        builder = get_architecture(archs[0])
    except KeyError as e:
        raise ConfigError(str(e.args[0])) from None
    return builder(raw_config, generation_config, strict)


def build_model_from_folder(model_dir: str, dtype: str, strict: bool = False) -> Tuple[object, Decoder]:
    raw = read_config_json(model_dir)
    cfg, spec = model_spec_for(raw, read_generation_config(model_dir), strict)
    model = Decoder(spec)
    shapes = {name: shape for name, (shape, _) in model.catalog().items()}
    model.bind(iter_checkpoint(model_dir, shapes, dtype, strict))
    return cfg, model


def build_model_from_config(raw_config: Mapping, seed: int, dtype: str, init_std: Optional[float] = None,
                            device_init: bool = False) -> Tuple[object, Decoder]:
    """Random weights without a folder.  ``device_init`` draws on the GPU (fast for large
    models; the values differ from the host generator's but depend on the seed alone)."""
    import torch
    cfg, spec = model_spec_for(raw_config)
    model = Decoder(spec)

    def gen():
        for name, t in random_tensors(model.catalog(), seed, init_std, "cuda" if device_init else "cpu"):
            yield name, (t.to(torch.float32) if dtype == "float32" else t)

    model.bind(gen())
    return cfg, model


def write_random_model(out_dir: str, raw_config: Mapping, seed: int, init_std: Optional[float] = None) -> str:
    """Write ``config.json`` + ``model.safetensors`` with random weights for ``raw_config``."""
    cfg, spec = model_spec_for(raw_config)
    model = Decoder(spec)
    return write_model_folder(out_dir, raw_config, model.catalog(), seed, init_std)
