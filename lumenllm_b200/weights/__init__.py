from .safetensors_io import SafetensorsError, read_header, write_file
from .loader import WeightError, check_against, load_weights, open_checkpoint
from .random_init import random_weights, write_random_model

__all__ = ["SafetensorsError", "read_header", "write_file", "WeightError", "check_against",
           "load_weights", "open_checkpoint", "random_weights", "write_random_model"]
