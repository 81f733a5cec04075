from .loader import check, discover, load_weights
from .random_init import random_tensors, write_random_model
from .spec import MATRIX, TABLE, VECTOR, TensorSpec, WeightPlan

__all__ = ["check", "discover", "load_weights", "random_tensors", "write_random_model",
           "MATRIX", "TABLE", "VECTOR", "TensorSpec", "WeightPlan"]
