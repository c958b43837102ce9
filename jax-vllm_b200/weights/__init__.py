from .loader import DamagedFile, WeightError, load_tensors, read_index, storage_dtype
from .random_init import random_tensor, random_tensors, tensor_seed, write_model_folder

__all__ = ["DamagedFile", "WeightError", "load_tensors", "read_index", "storage_dtype", "random_tensor", "random_tensors",
           "tensor_seed", "write_model_folder"]
