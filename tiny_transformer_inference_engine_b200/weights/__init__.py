from .loader import WeightError, read_safetensors, load_folder, place
from .random_init import random_tensors, write_random_model

__all__ = ["WeightError", "read_safetensors", "load_folder", "place", "random_tensors", "write_random_model"]
