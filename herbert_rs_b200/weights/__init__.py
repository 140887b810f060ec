"""Reading model folders and making random ones."""

from .loader import build_model, check_tensors, fill_model, load_model
from .random_init import random_model, random_tensor, random_tensors, write_random_model
from .safetensors_io import ModelFiles, SafeTensorsFile, save_file

__all__ = ["build_model", "check_tensors", "fill_model", "load_model", "random_model", "random_tensor",
           "random_tensors", "write_random_model", "ModelFiles", "SafeTensorsFile", "save_file"]
