"""From a model folder to a model on the device."""
from __future__ import annotations

import torch

from .. import ops
from ..config.registry import load_config
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..weights.loader import InitPolicy, load_tensors, random_tensors, write_model_folder

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not supported (bfloat16 or float32)") from None


def gguf_rename(model_path: str):
    """For a ``.gguf`` file the function that turns its tensor names into the checkpoint's."""
    from ..config.registry import architecture_for_gguf, is_gguf
    if not is_gguf(model_path):
        return None
    from ..weights.gguf_io import read_gguf
    return architecture_for_gguf(read_gguf(model_path)[0]).gguf.tensor_name


def load_model(model_path: str, dtype="bfloat16", device="cuda:0"):
    """Read config.json of a model folder (or the metadata of a ``.gguf`` file), pick the
    model by its architecture name, load the weights by tensor name.  Returns (typed config,
    DecoderModel)."""
    ops.require_gpu()
    runtime = Runtime(parse_dtype(dtype), torch.device(device))
    config, spec = load_config(model_path)
    model = DecoderModel(spec, runtime)
    rename = gguf_rename(model_path)
    tensors = load_tensors(model_path, model.tensor_specs(), runtime.dtype, runtime.device, rename=rename)
    model.bind(tensors)
    return config, model


def write_random_gguf(path: str, config, seed: int, policy: InitPolicy = InitPolicy(),
                      store: torch.dtype = torch.bfloat16) -> None:
    """The random-weights mode as one GGUF file (the same values as ``write_random_model``)."""
    from ..config.registry import architecture_for
    from ..weights.gguf_io import write_gguf
    obj = config.to_dict()
    arch = architecture_for(obj)
    if arch.gguf is None or arch.gguf.metadata_of is None:
        raise ValueError(f"architecture {arch.name} has no GGUF face")
    typed = arch.parse_config(obj)
    model = DecoderModel(arch.model_spec(typed), Runtime(store, torch.device("cpu")))
    tensors = random_tensors(model.tensor_specs(), seed, policy, store=store)
    write_gguf(path, arch.gguf.metadata_of(typed), [(arch.gguf.gguf_name_of(n), tensors[n]) for n in sorted(tensors)])


def write_random_model(model_dir: str, config, seed: int, policy: InitPolicy = InitPolicy(),
                       store: torch.dtype = torch.bfloat16) -> None:
    """The random-weights mode: write ``config.json`` and ``model.safetensors`` for a
    typed configuration and a seed (no GPU needed)."""
    from ..config.registry import architecture_for
    obj = config.to_dict()
    arch = architecture_for(obj)
    spec = arch.model_spec(arch.parse_config(obj))
    model = DecoderModel(spec, Runtime(store, torch.device("cpu")))
    tensors = random_tensors(model.tensor_specs(), seed, policy, store=store)
    write_model_folder(model_dir, obj, tensors)


def random_model_on_device(config, seed: int, dtype="bfloat16", device="cuda:0",
                           policy: InitPolicy = InitPolicy(norm_jitter=0.0)):
    """A model with seeded random weights made directly on the device (benchmarks)."""
    from ..config.registry import architecture_for
    from ..weights.loader import kept_dtype
    ops.require_gpu()
    runtime = Runtime(parse_dtype(dtype), torch.device(device))
    obj = config.to_dict()
    arch = architecture_for(obj)
    spec = arch.model_spec(arch.parse_config(obj))
    model = DecoderModel(spec, runtime)
    specs = model.tensor_specs()
    raw = random_tensors(specs, seed, policy, store=torch.bfloat16, device=runtime.device)
    tensors = {n: t.to(kept_dtype(specs[n], t.dtype, runtime.dtype)).contiguous() for n, t in raw.items()}
    model.bind(tensors)
    return model
