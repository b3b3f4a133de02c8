from .loader import WeightError, WeightSpec, check_weights, load_weights
from .nnis_directory import NnisDirectoryError, write_nnis_directory
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightError", "WeightSpec", "check_weights", "load_weights", "random_tensors", "write_random_model",
           "NnisDirectoryError", "write_nnis_directory", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
