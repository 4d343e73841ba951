from .loader import (INT_TABLE, KEEP32, MATRIX, ParamSpec, WeightError, check_against_specs, load_state,
                     state_from_tensors)
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_shards, write_safetensors

__all__ = ["INT_TABLE", "KEEP32", "MATRIX", "ParamSpec", "WeightError", "check_against_specs", "load_state",
           "state_from_tensors", "random_tensors", "write_model_folder", "SafetensorsError",
           "SafetensorsFile", "open_model_shards", "write_safetensors"]
