"""Weights: safetensors by tensor name, the needed-versus-held check, random initialisation."""
from .loader import TensorNeed, WeightsError, check, held_dtype, load, load_folder
from .random_init import RandomInit, make_tensor, make_tensors, write_model_folder
from .safetensors_io import (SafetensorsError, TensorSource, open_folder, read_header, write_file,
                             write_file_streaming)

__all__ = ["TensorNeed", "WeightsError", "check", "held_dtype", "load", "load_folder", "RandomInit",
           "make_tensor", "make_tensors", "write_model_folder", "SafetensorsError", "TensorSource",
           "open_folder", "read_header", "write_file", "write_file_streaming"]
