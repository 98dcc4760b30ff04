from .model_config import (
    ConfigError, DenseDecoderConfig, Llama3RopeScaling, config_from_hf_dict,
    read_config_json, read_generation_config,
)
from .spec import PartSpec, LayerSpec, RunEntry, ModelSpec, default_run_list
from .engine_config import EngineConfig

__all__ = [
    "ConfigError", "DenseDecoderConfig", "Llama3RopeScaling", "config_from_hf_dict",
    "read_config_json", "read_generation_config", "PartSpec", "LayerSpec", "RunEntry",
    "ModelSpec", "default_run_list", "EngineConfig",
]
