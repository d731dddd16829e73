from .loader import (
    WeightError,
    check_names_and_shapes,
    find_safetensors_files,
    load_weights,
    stored_dtype,
)
from .random_weights import random_tensor, random_tensors, write_random_model

__all__ = [
    "WeightError", "check_names_and_shapes", "find_safetensors_files", "load_weights",
    "random_tensor", "random_tensors", "stored_dtype", "write_random_model",
]
