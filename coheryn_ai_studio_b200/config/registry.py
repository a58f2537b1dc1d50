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
from typing import Any, Callable, Dict, Tuple

from .qwen2 import ConfigError, Qwen2Config, qwen2_model_spec, read_config_json
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]   # config.json object -> typed config
    model_spec: Callable[[Any], ModelSpec]          # typed config -> layer layout


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, model_spec, *, replace: bool = False) -> None:
    if not name:
        raise ValueError("an architecture needs a non-empty name")
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, model_spec)


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


def load_config(model_dir: str):
    """Read ``model_dir/config.json``; return (typed config, ModelSpec)."""
    obj = read_config_json(os.path.join(model_dir, "config.json"))
    arch = architecture_for(obj)
    config = arch.parse_config(obj)
    spec = arch.model_spec(config)
    spec.validate()
    return config, spec


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_model_spec)
