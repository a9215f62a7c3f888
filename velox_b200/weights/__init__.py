from .loader import Checkpoint, WeightError, WeightStore, check_checkpoint, storage_dtype
from .random_init import random_state_dict, random_tensor, tensor_seed, write_random_model

__all__ = [
    "Checkpoint",
    "WeightError",
    "WeightStore",
    "check_checkpoint",
    "random_state_dict",
    "random_tensor",
    "storage_dtype",
    "tensor_seed",
    "write_random_model",
]
