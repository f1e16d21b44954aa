from .loader import CheckpointMismatch, load_weights
from .random_init import random_tensors, write_model_folder

__all__ = ["CheckpointMismatch", "load_weights", "random_tensors", "write_model_folder"]
