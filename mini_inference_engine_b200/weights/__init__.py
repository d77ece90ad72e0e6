from .loader import TensorSpec, WeightError, check_and_bind, read_model_folder, storage_dtype
from .random_init import random_state, random_tensor, write_model_folder
from .safetensors_io import SafetensorsError, read_file, write_file

__all__ = ["TensorSpec", "WeightError", "check_and_bind", "read_model_folder", "storage_dtype",
           "random_state", "random_tensor", "write_model_folder", "SafetensorsError", "read_file", "write_file"]
