from .loader import WeightsError, kept_dtype, match_names, open_checkpoint
from .random_init import random_source, random_tensor, write_random_model
from .safetensors_io import Checkpoint, write_safetensors
from .tensors import TensorSpec

__all__ = [
    "Checkpoint", "TensorSpec", "WeightsError", "kept_dtype", "match_names", "open_checkpoint",
    "random_source", "random_tensor", "write_random_model", "write_safetensors",
]
