from .loader import WeightError, WeightFileError, expected_tensors, load_weights
from .random_init import random_weights_on_device, write_random_model

__all__ = ["WeightError", "WeightFileError", "expected_tensors", "load_weights", "random_weights_on_device", "write_random_model"]
