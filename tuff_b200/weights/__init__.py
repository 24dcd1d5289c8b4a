from .loader import WeightError, load_checkpoint
from .random_init import write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, write_safetensors

__all__ = ["WeightError", "load_checkpoint", "write_random_model", "ModelFiles", "SafetensorsError",
           "write_safetensors"]
