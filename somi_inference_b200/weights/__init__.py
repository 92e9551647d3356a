"""Weights: safetensors reading and writing, the checked loader, random model folders."""

from .loader import WeightError, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, save_safetensors

__all__ = ["WeightError", "load_tensors", "random_tensors", "write_random_model",
           "SafetensorsFile", "save_safetensors"]
