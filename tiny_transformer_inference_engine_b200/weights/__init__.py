from .loader import WeightError, read_safetensors, load_folder, place
from .random_init import random_tensors, write_random_model
from .convert import CheckpointError, convert_checkpoint

__all__ = ["WeightError", "read_safetensors", "load_folder", "place", "random_tensors", "write_random_model",
           "CheckpointError", "convert_checkpoint"]
