from .loader import WeightError, load_weights
from .random_init import random_tensor, random_weights, write_random_model
from .tensor_spec import TensorSpec

__all__ = ["TensorSpec", "WeightError", "load_weights", "random_tensor", "random_weights",
           "write_random_model"]
