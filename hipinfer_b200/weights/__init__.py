from .loader import (ParamSpec, WeightError, check_names, load_weights, random_weights, storage_dtype,
                     write_random_model)
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, save_safetensors

__all__ = ["ParamSpec", "WeightError", "check_names", "load_weights", "random_weights", "storage_dtype",
           "write_random_model", "ModelFiles", "SafetensorsError", "SafetensorsFile", "save_safetensors"]
