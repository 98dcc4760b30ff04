from .safetensors_io import CheckpointFiles, SafetensorsError, read_header, write_safetensors
from .loader import WeightError, check_catalog, load_checkpoint, iter_checkpoint, convert_stored
from .random_init import random_tensor, random_tensors, write_model_folder

__all__ = [
    "CheckpointFiles", "SafetensorsError", "read_header", "write_safetensors", "WeightError",
    "check_catalog", "load_checkpoint", "iter_checkpoint", "convert_stored", "random_tensor",
    "random_tensors", "write_model_folder",
]
