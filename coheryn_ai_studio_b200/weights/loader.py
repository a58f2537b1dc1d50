"""Weights by tensor name: loading from safetensors and a seeded random-weights mode.

Loading checks the whole set at once, as the reference's graph validator does
(crates/coheryn-engine/src/compat.rs:161-221: exact tensor set, exact shapes, extra
tensors refused), and reports every missing tensor, every unexpected tensor and every
wrong shape in ONE error.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .safetensors_io import TensorReader, index_model_dir, write_file
from .spec import TensorSpec


class WeightError(ValueError):
    """The checkpoint does not hold exactly the tensors the model needs."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, found, wanted)
        self.wrong_dtype = list(wrong_dtype)      # (name, found, wanted kind)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, found, wanted in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, the model needs {list(wanted)}")
        for name, found, wanted in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {found}, the model needs {wanted}")
        super().__init__("\n".join(lines))


def kept_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device (see :class:`TensorSpec`)."""
    if spec.role == "int_table":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.role == "vector" and stored == torch.float32:
        return torch.float32
    return compute


def check_against(expected: Dict[str, TensorSpec], entries) -> None:
    missing = [n for n, s in expected.items() if n not in entries and not s.optional]
    unexpected = [n for n in entries if n not in expected]
    wrong_shape, wrong_dtype = [], []
    for n, s in expected.items():
        e = entries.get(n)
        if e is None:
            continue
        if tuple(e.shape) != tuple(s.shape):
            wrong_shape.append((n, tuple(e.shape), tuple(s.shape)))
        is_int = e.dtype == torch.int32
        if is_int != (s.role == "int_table"):
            wrong_dtype.append((n, str(e.dtype).replace("torch.", ""),
                                "int32" if s.role == "int_table" else "a floating type"))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)


def index_model(model_path: str, rename=None):
    """Tensor index by checkpoint name of a folder of safetensors, or of a ``.gguf`` file whose
    tensor names ``rename`` turns into the checkpoint's."""
    if not os.path.isfile(model_path):
        return index_model_dir(model_path)
    from .gguf_io import read_gguf
    entries = {}
    for name, e in read_gguf(model_path)[1].items():
        new = rename(name) if rename is not None else name
        if new in entries:
            raise ValueError(f"tensor {name} and another both map to {new}")
        entries[new] = e
    return entries


def load_tensors(model_path: str, expected: Dict[str, TensorSpec], compute: torch.dtype,
                 device, rename=None) -> Dict[str, torch.Tensor]:
    """Read every expected tensor, cast it to the dtype it is kept in, move it to
    ``device`` (``model_path`` and ``rename`` as for :func:`index_model`).  Raises
    :class:`WeightError` before reading any payload if the set of names or any shape is wrong."""
    entries = index_model(model_path, rename)
    check_against(expected, entries)
    reader = TensorReader(entries)
    out: Dict[str, torch.Tensor] = {}
    try:
        for name, spec in expected.items():
            if name not in entries:
                continue
            t = reader.read(name)
            if t.dtype != torch.int32 and not torch.isfinite(t.float()).all():
                raise ValueError(f"tensor {name} holds a non-finite value")
            out[name] = t.to(kept_dtype(spec, t.dtype, compute)).to(device).contiguous()
    finally:
        reader.close()
    return out


@dataclass(frozen=True)
class InitPolicy:
    """Standard deviations of the random-weights mode."""

    matrix_std: float = 0.02
    bias_std: float = 0.02
    norm_jitter: float = 0.01


def random_tensors(expected: Dict[str, TensorSpec], seed: int, policy: InitPolicy,
                   store: torch.dtype = torch.bfloat16, device="cpu",
                   vector_dtype: Optional[torch.dtype] = torch.float32) -> Dict[str, torch.Tensor]:
    """Seeded random values for every expected tensor: each element is a function of
    (seed, tensor name, element index) alone (see :mod:`.seeded`), so the result is the same on
    the host and on the device, for a whole model or for one tensor of it.  Values are made in
    float32 and rounded to ``store``; norm weights are kept in ``vector_dtype`` when given, so a
    folder written from them exercises the "stored in 32-bit stays 32-bit" rule."""
    from .seeded import seeded_tensor
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.role == "int_table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        dt = store
        if spec.init == "norm" and vector_dtype is not None:
            dt = vector_dtype
        if spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=dt, device=device)
            continue
        try:
            mean, deviation = {"normal": (0.0, policy.matrix_std), "bias": (0.0, policy.bias_std),
                               "norm": (1.0, policy.norm_jitter)}[spec.init]
        except KeyError:
            raise ValueError(f"tensor {name}: unknown init {spec.init!r}") from None
        out[name] = seeded_tensor(seed, name, spec.shape, mean, deviation, dtype=dt, device=device)
    return out


def write_model_folder(model_dir: str, config_object: dict, tensors: Dict[str, torch.Tensor]) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config_object, f, indent=1, sort_keys=True)
    write_file(os.path.join(model_dir, "model.safetensors"),
               [(n, tensors[n]) for n in sorted(tensors)], metadata={"format": "pt"})
