from .loader import WeightError, load_weights
from .random_init import materialize_random, write_random_model

__all__ = ["WeightError", "load_weights", "materialize_random", "write_random_model"]
