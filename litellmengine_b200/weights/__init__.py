"""Weights: the safetensors container, sources of tensors, binding by name."""
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors
from .loader import (DictSource, ParamSpec, RandomSource, SafetensorsSource, WeightError,
                     WeightSource, bind_weights, check_source, fetch_tensor,
                     write_random_model)

__all__ = ["SafetensorsError", "SafetensorsFile", "open_model_files", "write_safetensors",
           "DictSource", "ParamSpec", "RandomSource", "SafetensorsSource", "WeightError",
           "WeightSource", "bind_weights", "check_source", "fetch_tensor", "write_random_model"]
