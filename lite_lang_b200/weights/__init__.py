from .loader import Checkpoint, WeightError, check_against, load_weights
from .random_init import draw_tensor, random_fetch, write_random_model

__all__ = ["Checkpoint", "WeightError", "check_against", "load_weights", "draw_tensor", "random_fetch",
           "write_random_model"]
