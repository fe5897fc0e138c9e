"""Weights: safetensors by tensor name, and the random-weights mode."""

from .loader import TensorIndex, WeightError, check_inventory, load_weights
from .random_init import random_tensors, write_random_model

__all__ = ["TensorIndex", "WeightError", "check_inventory", "load_weights", "random_tensors", "write_random_model"]
