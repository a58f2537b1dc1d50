from .gguf_io import GgufError, read_gguf, write_gguf
from .loader import (InitPolicy, WeightError, check_against, index_model, kept_dtype, load_tensors, random_tensors,
                     write_model_folder)
from .safetensors_io import SafetensorsError, TensorReader, index_model_dir, read_header, write_file
from .spec import TensorSpec

__all__ = ["GgufError", "read_gguf", "write_gguf", "index_model", "InitPolicy", "WeightError", "check_against", "kept_dtype", "load_tensors",
           "random_tensors", "write_model_folder", "SafetensorsError", "TensorReader",
           "index_model_dir", "read_header", "write_file", "TensorSpec"]
