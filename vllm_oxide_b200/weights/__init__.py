from .loader import TensorSpec, WeightsError, check_specs, kept_dtype, load_checked
from .random_init import random_weights, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, resolve_shards, write_safetensors

__all__ = ["TensorSpec", "WeightsError", "check_specs", "kept_dtype", "load_checked", "random_weights",
           "write_model_folder", "SafetensorsError", "SafetensorsFile", "resolve_shards", "write_safetensors"]
