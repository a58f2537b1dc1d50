from .loading import load_model, parse_dtype, random_model_on_device, write_random_model
from .step import OutOfPages, StepEntry, StepRunner

__all__ = ["load_model", "parse_dtype", "random_model_on_device", "write_random_model",
           "OutOfPages", "StepEntry", "StepRunner"]
