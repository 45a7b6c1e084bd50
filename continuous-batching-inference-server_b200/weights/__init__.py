from .safetensors_io import WeightsError, read_safetensors, write_safetensors
from .loader import TensorDecl, check_tensors, read_model_tensors
from .random_init import InitScheme, random_tensors, write_model_folder

__all__ = ["WeightsError", "read_safetensors", "write_safetensors", "TensorDecl", "check_tensors",
           "read_model_tensors", "InitScheme", "random_tensors", "write_model_folder"]
