from .loader import TensorRequest, TensorSource, WeightError, WeightStore, storage_dtype
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightFileError, open_model_files, write_safetensors

__all__ = ["TensorRequest", "TensorSource", "WeightError", "WeightStore", "storage_dtype", "random_tensor",
           "random_tensors", "write_random_model", "SafetensorsFile", "WeightFileError", "open_model_files",
           "write_safetensors"]
