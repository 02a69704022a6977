"""Weights: the safetensors container, loading by tensor name, random weights."""
from .safetensors import Checkpoint, SafetensorsFile, SafetensorsFormatError, save_file
from .loader import (WeightError, WeightSpec, load_weights, random_weights, write_model_folder,
                     write_random_model)

__all__ = ["Checkpoint", "SafetensorsFile", "SafetensorsFormatError", "save_file", "WeightError",
           "WeightSpec", "load_weights", "random_weights", "write_model_folder", "write_random_model"]
