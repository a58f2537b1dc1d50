from .engine import Engine, GenerationResult
from .loading import load_model, parse_dtype, random_model_on_device, write_random_gguf, write_random_model
from .scheduler import Request, RequestRefused, Scheduled, Scheduler
from .step import OutOfPages, StepEntry, StepRunner

__all__ = ["Engine", "GenerationResult", "load_model", "parse_dtype", "random_model_on_device",
           "write_random_model", "write_random_gguf", "Request", "RequestRefused", "Scheduled", "Scheduler", "OutOfPages",
           "StepEntry", "StepRunner"]
