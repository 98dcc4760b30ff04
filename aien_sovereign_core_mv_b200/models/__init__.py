from . import llama_qwen3  # noqa: F401  (registers the architectures)
from .decoder import Decoder
from .loading import build_model_from_folder, build_model_from_config, model_spec_for

__all__ = ["Decoder", "build_model_from_folder", "build_model_from_config", "model_spec_for"]
