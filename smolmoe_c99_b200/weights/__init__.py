"""Weights: the safetensors container, binding by tensor name, and the random-weights mode."""
from .loader import WeightsError, load_weights, stored_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_checkpoint, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightsError", "load_weights", "open_checkpoint",
           "random_tensors", "stored_dtype", "write_random_model", "write_safetensors"]
