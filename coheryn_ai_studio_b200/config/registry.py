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
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]   # config.json object -> typed config
    model_spec: Callable[[Any], ModelSpec]          # typed config -> layer layout
    gguf: Optional[GgufFace] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, model_spec, *, gguf: Optional[GgufFace] = None,
                          replace: bool = False) -> None:
    if not name:
        raise ValueError("an architecture needs a non-empty name")
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    if gguf is not None and any(a.gguf is not None and a.gguf.name == gguf.name and a.name != name
                                for a in _ARCHITECTURES.values()):
        raise ValueError(f"GGUF architecture {gguf.name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, model_spec, gguf)


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


def load_config(model_path: str):
    """Read ``model_path/config.json``, or the metadata of a ``.gguf`` file; return (typed
    config, ModelSpec)."""
    if is_gguf(model_path):
        from ..weights.gguf_io import read_gguf
        meta, entries = read_gguf(model_path)
        arch = architecture_for_gguf(meta)
        config = arch.gguf.parse_metadata(meta, entries.keys())
    else:
        obj = read_config_json(os.path.join(model_path, "config.json"))
        arch = architecture_for(obj)
        config = arch.parse_config(obj)
    spec = arch.model_spec(config)
    spec.validate()
    return config, spec


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_model_spec,
                      gguf=GgufFace("qwen2", qwen2_config_from_gguf, qwen2_gguf_tensor_name,
                                    qwen2_gguf_metadata, qwen2_gguf_name_of))
