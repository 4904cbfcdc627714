from .loader import WeightsError, bind_tensors, expected_tensors, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["WeightsError", "bind_tensors", "expected_tensors", "load_tensors", "random_tensors",
           "write_random_model", "SafetensorsFile", "write_safetensors"]
