from .errors import WeightsError
from .loader import check, keep_dtype, load_checked
from .random_init import random_tensors, write_model_dir
from .safetensors_io import read_dir, read_file, write_file

__all__ = ["WeightsError", "check", "keep_dtype", "load_checked", "random_tensors", "write_model_dir", "read_dir",
           "read_file", "write_file"]
