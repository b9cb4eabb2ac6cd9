from .loader import WeightError, check_names, load_checkpoint, place
from .random_init import random_checkpoint, random_tensor, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightError", "check_names", "load_checkpoint",
           "open_model_files", "place", "random_checkpoint", "random_tensor", "write_model_folder",
           "write_safetensors"]
