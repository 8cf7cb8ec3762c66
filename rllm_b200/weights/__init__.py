from .loader import WeightMismatchError, load_checked
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightFileError, write_safetensors

__all__ = ["WeightMismatchError", "load_checked", "random_tensors", "write_random_model",
           "SafetensorsFile", "WeightFileError", "write_safetensors"]
