from .loader import WeightsError, load_model_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, save_safetensors

__all__ = ["WeightsError", "load_model_tensors", "random_tensors", "write_random_model", "SafetensorsError",
           "SafetensorsFile", "save_safetensors"]
