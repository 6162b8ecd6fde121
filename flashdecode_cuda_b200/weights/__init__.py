"""Checkpoints by tensor name, their checks and the random-weights mode."""

from .loader import (WeightError, cast, check, load_checkpoint, random_tensor, random_tensors,
                     write_model_folder)
from .safetensors_io import SafetensorsError, read_file, read_folder, write_file
from .spec import TensorSpec

__all__ = ["TensorSpec", "WeightError", "SafetensorsError", "check", "cast", "load_checkpoint",
           "random_tensor", "random_tensors", "write_model_folder", "read_file", "read_folder", "write_file"]
