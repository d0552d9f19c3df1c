from .loader import (DictSource, FolderSource, TensorSource, WeightError, check_names_and_shapes,
                     load_params, place)
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["DictSource", "FolderSource", "TensorSource", "WeightError", "check_names_and_shapes",
           "load_params", "place", "random_tensor", "random_tensors", "write_random_model",
           "Checkpoint", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
