"""Weight files: safetensors reader/writer, the by-name loader, random weights."""
from .loader import WeightError, load_weights
from .random_init import write_random_model
from .safetensors import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightError", "load_weights",
           "write_random_model", "write_safetensors"]
