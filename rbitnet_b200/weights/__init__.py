from .safetensors_io import WeightError, read_safetensors, read_model_tensors, write_safetensors
from .loader import check_tensors, load_checked
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["WeightError", "read_safetensors", "read_model_tensors", "write_safetensors",
           "check_tensors", "load_checked", "random_tensor", "random_tensors", "write_random_model"]
