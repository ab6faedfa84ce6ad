from .loader import (WeightError, check_names_and_shapes, init_random_weights, load_model_weights,
                     random_tensor, write_random_model)
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["WeightError", "check_names_and_shapes", "init_random_weights", "load_model_weights",
           "random_tensor", "write_random_model", "SafetensorsError", "SafetensorsFile",
           "open_model_files", "write_safetensors"]
