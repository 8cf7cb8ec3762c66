from .loader import WeightMismatchError, load_checked, weight_files
from .random_init import random_tensors, write_random_model, write_sharded
from .safetensors_io import SafetensorsFile, WeightFileError, write_safetensors

__all__ = ["WeightMismatchError", "load_checked", "weight_files", "write_sharded", "random_tensors", "write_random_model",
           "SafetensorsFile", "WeightFileError", "write_safetensors"]
