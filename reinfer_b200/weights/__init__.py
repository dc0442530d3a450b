from .params import ParamSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_tensors, write_safetensors
from .loader import WeightError, load_state, random_state, write_random_model

__all__ = ["ParamSpec", "SafetensorsError", "SafetensorsFile", "open_model_tensors",
           "write_safetensors", "WeightError", "load_state", "random_state", "write_random_model"]
