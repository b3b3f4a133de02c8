from .loader import WeightError, WeightSpec, check_weights, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightError", "WeightSpec", "check_weights", "load_weights", "random_tensors", "write_random_model",
           "SafetensorsError", "SafetensorsFile", "write_safetensors"]
