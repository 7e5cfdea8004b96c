from .loader import TensorReq, WeightError, check_tensors, load_checkpoint, read_model_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, read_file, read_header, write_file

__all__ = ["TensorReq", "WeightError", "check_tensors", "load_checkpoint", "read_model_tensors",
           "random_tensors", "write_random_model", "SafetensorsError", "read_file", "read_header", "write_file"]
