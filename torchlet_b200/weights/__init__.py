from .loader import LazyCheckpoint, WeightsError, check_and_normalise, load_checkpoint, read_safetensors
from .random_init import random_tensors, write_random_model

__all__ = ["LazyCheckpoint", "WeightsError", "check_and_normalise", "load_checkpoint", "read_safetensors", "random_tensors",
           "write_random_model"]
