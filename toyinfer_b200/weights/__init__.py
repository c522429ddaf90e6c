"""Checkpoints: safetensors by name, and random weights."""
from .loader import WeightError, load_parameters
from .random_init import draw, random_parameters, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model, write_safetensors

__all__ = [
    "WeightError", "load_parameters", "draw", "random_parameters", "write_model_folder",
    "SafetensorsError", "SafetensorsFile", "open_model", "write_safetensors",
]
