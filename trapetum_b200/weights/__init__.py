from .loader import TensorSpec, WeightError, load_tensors, random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightFileError, open_model_files, write_safetensors

__all__ = ["SafetensorsFile", "TensorSpec", "WeightError", "WeightFileError", "load_tensors", "open_model_files",
           "random_tensors", "write_random_model", "write_safetensors"]
