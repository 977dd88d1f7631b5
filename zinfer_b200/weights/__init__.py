from .checkpoint import Checkpoint, CheckpointError, write_sharded
from .loader import WeightsError, check_against, kept_dtype, load_tensors
from .random_init import random_tensor, random_tensors, write_model_dir
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorInfo, write_safetensors

__all__ = ["Checkpoint", "CheckpointError", "SafetensorsError", "SafetensorsFile", "TensorInfo", "WeightsError",
           "check_against", "kept_dtype", "load_tensors", "random_tensor", "random_tensors", "write_model_dir",
           "write_safetensors", "write_sharded"]
