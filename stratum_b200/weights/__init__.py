from .loader import WeightError, check_tensors, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["WeightError", "check_tensors", "load_weights", "random_tensors", "write_random_model",
           "SafetensorsError", "SafetensorsFile", "open_model_files", "write_safetensors"]
