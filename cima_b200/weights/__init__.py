from .loader import (CheckpointTensors, RandomTensors, TensorSource, TensorSpec, WeightError, load_tensors,
                     stored_to_kept, tensor_names)
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, parse_header, write_safetensors

__all__ = ["CheckpointTensors", "RandomTensors", "TensorSource", "TensorSpec", "WeightError", "load_tensors", "stored_to_kept", "tensor_names", "random_tensor", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "open_model_files", "parse_header",
           "write_safetensors"]
