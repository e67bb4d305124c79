from .loader import TensorSource, WeightError, check, load_into
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["TensorSource", "WeightError", "check", "load_into", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
