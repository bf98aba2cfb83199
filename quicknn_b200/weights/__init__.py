"""Weights: safetensors by tensor name, the precision policy, random models."""
from .loader import WeightError, check_names_and_shapes, check_state_dict, load_named_tensors, place
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorDirectory, write_safetensors

__all__ = ["WeightError", "check_names_and_shapes", "check_state_dict", "load_named_tensors", "place",
           "random_tensors", "write_model_folder", "SafetensorsError", "SafetensorsFile", "TensorDirectory",
           "write_safetensors"]
