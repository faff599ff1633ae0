from .loader import WeightError, check_and_cast, load_model, read_hf_config, read_safetensors, resolve_dtype
from .random_init import random_tensors, write_model_folder, write_random_stub

__all__ = ["WeightError", "check_and_cast", "load_model", "read_hf_config", "read_safetensors", "resolve_dtype",
           "random_tensors", "write_model_folder", "write_random_stub"]
