from .loader import WeightError, check_tensors, load_weights
from .random_init import fill_random, random_tensor, write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightError", "check_tensors", "load_weights", "fill_random", "random_tensor", "write_random_model",
           "ModelFiles", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
