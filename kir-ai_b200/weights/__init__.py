"""Reading model folders (safetensors by tensor name) and making random ones."""
from .loader import WeightError, WeightSource, from_tensors, open_checked
from .random_init import random_tensors, write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightError", "WeightSource", "from_tensors", "open_checked", "random_tensors", "write_random_model",
           "ModelFiles", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
