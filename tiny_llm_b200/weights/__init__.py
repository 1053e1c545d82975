from .errors import WeightError
from .loader import (AS_STORED, COMPUTE, FLOAT32, INT32, ShardedSafetensors, WeightSpec, check_against, load_state,
                     open_source)
from .random_init import random_state, write_random_model
from .safetensors_io import SafetensorsFile, save_safetensors

__all__ = ["WeightError", "WeightSpec", "COMPUTE", "FLOAT32", "INT32", "AS_STORED", "check_against",
           "load_state", "open_source", "ShardedSafetensors", "random_state", "write_random_model", "SafetensorsFile",
           "save_safetensors"]
