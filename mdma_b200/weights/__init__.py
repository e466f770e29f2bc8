from .loader import (WeightsError, check_entries, load_tensors, open_model_files, resident_dtype,
                     stored_dtypes)
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import CheckpointError, SafetensorsFile, read_header, write_safetensors

__all__ = ["WeightsError", "CheckpointError", "SafetensorsFile", "check_entries", "load_tensors",
           "open_model_files", "random_tensor", "random_tensors", "read_header", "resident_dtype", "stored_dtypes",
           "write_random_model", "write_safetensors"]
