from .loader import CheckpointError, check_layout, checkpoint_index, load_parameters
from .random_init import random_checkpoint_tensors, random_parameters, write_random_model

__all__ = [
    "CheckpointError", "check_layout", "checkpoint_index", "load_parameters",
    "random_checkpoint_tensors", "random_parameters", "write_random_model",
]
