"""Weights: safetensors by tensor name, and seeded random weights."""
from .safetensors_io import SafetensorsFile, TensorEntry, write_safetensors
from .loader import TensorDecl, bind_tensors, open_checkpoint, target_dtype
from .random_init import InitScales, random_tensors, write_model_folder

__all__ = ["SafetensorsFile", "TensorEntry", "write_safetensors", "TensorDecl", "bind_tensors",
           "open_checkpoint", "target_dtype", "InitScales", "random_tensors", "write_model_folder"]
