"""One registry from an architecture's name (``architectures[0]`` of config.json) to
its typed configuration and to the function that lays its layers out.

Semantics follow the reference's adapter registry
(crates/coheryn-engine/src/adapters.rs:59-117, docs/ADAPTERS.md): an empty or duplicate
id is refused at registration, an unknown architecture is an error that lists what is
registered, and there is no fallback to another adapter after a failure.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

from .qwen2 import (ConfigError, Qwen2Config, qwen2_config_from_gguf, qwen2_gguf_metadata, qwen2_gguf_name_of,
                    qwen2_gguf_tensor_name, qwen2_model_spec, read_config_json)
from .spec import ModelSpec


@dataclass(frozen=True)
class GgufFace:
    """How an architecture reads (and writes) a GGUF file: its ``general.architecture`` id,
    metadata -> typed config, GGUF tensor name -> checkpoint name, and the two inverses."""
    name: str
    parse_metadata: Callable[[Dict[str, Any], Any], Any]
    tensor_name: Callable[[str], str]
    metadata_of: Optional[Callable[[Any], Dict[str, Any]]] = None
    gguf_name_of: Optional[Callable[[str], str]] = None


@dataclass(frozen=True)
class Capabilities:
    """What an adapter can do, as metadata (crates/coheryn-engine/src/adapters.rs:11-21: adapter,
    architecture, format, text_generation, images, managed_api, continuous_batching,
    qualification).  ``formats`` and ``dtypes`` list what this engine loads and computes in;
    ``paged_kv`` and the byte counts come from what the model's mixers ask of the cache."""
    adapter: str
    architecture: str
    formats: Tuple[str, ...]
    dtypes: Tuple[str, ...]
    text_generation: bool
    images: bool
    continuous_batching: bool
    paged_kv: bool
    kv_bytes_per_token: Dict[str, int]               # by compute dtype
    fixed_state_bytes_per_request: int
    qualification: str


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]   # config.json object -> typed config
    model_spec: Callable[[Any], ModelSpec]          # typed config -> layer layout
    gguf: Optional[GgufFace] = None
    adapter_id: str = ""

    def describe(self, config) -> Dict[str, Any]:
        """Metadata only, nothing is loaded (crates/coheryn-engine/src/adapters.rs:39-58
        ``TextAdapter::describe``): the capabilities, the configuration, the layer layout in
        numbers and what one token and one request cost in the cache."""
        import torch

        from ..parts.base import FixedState, PagedKV, Runtime
        from ..parts.model import DecoderModel
        spec = self.model_spec(config)
        spec.validate()
        model = DecoderModel(spec, Runtime(torch.bfloat16, torch.device("cpu")))
        needs = model.cache_requirements()
        kv_elements = sum(2 * n.num_kv_heads * n.head_dim for n in needs if isinstance(n, PagedKV))
        state_bytes = 0
        for n in needs:
            if isinstance(n, FixedState):
                count = 1
                for d in n.shape:
                    count *= int(d)
                state_bytes += count * torch.empty((), dtype=n.dtype).element_size()
        specs = model.tensor_specs()
        parameters = 0
        for ts in specs.values():
            count = 1
            for d in ts.shape:
                count *= int(d)
            parameters += count
        caps = Capabilities(
            adapter=self.adapter_id or f"{self.name.lower()}-b200-v1", architecture=self.name,
            formats=("safetensors",) + (("gguf",) if self.gguf is not None else ()),
            dtypes=("bfloat16", "float32"), text_generation=True, images=False, continuous_batching=True,
            paged_kv=kv_elements > 0, kv_bytes_per_token={"bfloat16": 2 * kv_elements, "float32": 4 * kv_elements},
            fixed_state_bytes_per_request=state_bytes, qualification="random-weights parity with the plain implementation")
        windows = sorted({n.window for n in needs if isinstance(n, PagedKV) and n.window is not None})
        from dataclasses import asdict
        return {
            "capabilities": asdict(caps),
            "config": config.to_dict() if hasattr(config, "to_dict") else None,
            "layers": len(spec.layers), "schedule_entries": len(spec.schedule),
            "cache_entries": sum(1 for n in needs if n is not None), "attention_windows": windows,
            "tensors": len(specs), "parameters": parameters,
            "context": spec.max_positions, "vocabulary": spec.vocab_size,
        }


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, model_spec, *, gguf: Optional[GgufFace] = None,
                          replace: bool = False, adapter_id: str = "") -> None:
    if not name:
        raise ValueError("an architecture needs a non-empty name")
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    if gguf is not None and any(a.gguf is not None and a.gguf.name == gguf.name and a.name != name
                                for a in _ARCHITECTURES.values()):
        raise ValueError(f"GGUF architecture {gguf.name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, model_spec, gguf, adapter_id)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_for(config_object: Dict[str, Any]) -> Architecture:
    archs = config_object.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError("config.json must name exactly one architecture in 'architectures'")
    try:
        return _ARCHITECTURES[archs[0]]
    except KeyError:
        raise ConfigError(
            f"architecture {archs[0]!r} is not registered (registered: "
            f"{', '.join(registered_architectures()) or 'none'})") from None


def is_gguf(model_path: str) -> bool:
    return os.path.isfile(model_path) and model_path.lower().endswith(".gguf")


def architecture_for_gguf(metadata: Dict[str, Any]) -> Architecture:
    name = metadata.get("general.architecture")
    for arch in _ARCHITECTURES.values():
        if arch.gguf is not None and arch.gguf.name == name:
            return arch
    known = sorted(a.gguf.name for a in _ARCHITECTURES.values() if a.gguf is not None)
    raise ConfigError(f"GGUF architecture {name!r} is not registered (registered: {', '.join(known) or 'none'})")


def describe_model(model_path: str) -> Dict[str, Any]:
    """``Architecture.describe`` for a model folder or ``.gguf`` file (reads no tensor payload)."""
    arch, config = _arch_and_config(model_path)
    return arch.describe(config)


def load_config(model_path: str):
    """Read ``model_path/config.json``, or the metadata of a ``.gguf`` file; return (typed
    config, ModelSpec)."""
    arch, config = _arch_and_config(model_path)
    spec = arch.model_spec(config)
    spec.validate()
    return config, spec


def _arch_and_config(model_path: str):
    if is_gguf(model_path):
        from ..weights.gguf_io import read_gguf
        meta, entries = read_gguf(model_path)
        arch = architecture_for_gguf(meta)
        config = arch.gguf.parse_metadata(meta, entries.keys())
    else:
        obj = read_config_json(os.path.join(model_path, "config.json"))
        arch = architecture_for(obj)
        config = arch.parse_config(obj)
    return arch, config


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_model_spec,
                      gguf=GgufFace("qwen2", qwen2_config_from_gguf, qwen2_gguf_tensor_name,
                                    qwen2_gguf_metadata, qwen2_gguf_name_of),
                      adapter_id="qwen2-b200-v1")
