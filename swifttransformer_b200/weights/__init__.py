from .loader import WeightError, load_named_tensors
from .random_init import random_named_tensors, write_random_checkpoint
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .spec import GAIN, INT_TABLE, MATRIX, TABLE, VECTOR, ParamSpec

__all__ = ["GAIN", "INT_TABLE", "MATRIX", "TABLE", "VECTOR", "ParamSpec", "SafetensorsError",
           "SafetensorsFile", "WeightError", "load_named_tensors", "random_named_tensors",
           "write_random_checkpoint", "write_safetensors"]
