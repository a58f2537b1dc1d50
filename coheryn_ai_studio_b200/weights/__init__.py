from .loader import (InitPolicy, WeightError, check_against, kept_dtype, load_tensors, random_tensors,
                     write_model_folder)
from .safetensors_io import SafetensorsError, TensorReader, index_model_dir, read_header, write_file
from .spec import TensorSpec

__all__ = ["InitPolicy", "WeightError", "check_against", "kept_dtype", "load_tensors",
           "random_tensors", "write_model_folder", "SafetensorsError", "TensorReader",
           "index_model_dir", "read_header", "write_file", "TensorSpec"]
