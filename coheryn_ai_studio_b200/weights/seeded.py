"""Seeded random weights as a pure function of (seed, tensor name, element index).

The reference tests patch synthetic weights into a file (crates/coheryn-engine/tests/common/
mod.rs:47-251); here a model of any size is made from a seed, and every holder of that seed
- a folder written on the host, a model made directly on the device, a plain
implementation that wants three rows of the embedding - gets the same bits:

    key      = seed XOR fnv1a64(tensor name)
    draw(n)  = n-th output of SplitMix64 started at key (the sampler's constants,
               crates/coheryn-engine/src/sampling.rs:123-130)
    value(i) = float32(mean + deviation * BoxMuller(draw(2i+1), draw(2i+2)))

The arithmetic is in ``csrc/seeded_values.h`` (host C++ and the CUDA kernel include the same
header; logarithm and cosine are spelled out in IEEE double operations so that no maths
library's last bit enters).  A bfloat16 tensor holds the float32 value rounded to nearest even.
"""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

from ..csrc import build

_KINDS = {torch.float32: 0, torch.bfloat16: 1}
_host = None


def _host_lib():
    global _host
    if _host is None:
        lib = build.host_library()
        lib.coheryn_seeded_key.restype = ctypes.c_ulonglong
        lib.coheryn_seeded_key.argtypes = [ctypes.c_ulonglong, ctypes.c_char_p, ctypes.c_int]
        lib.coheryn_seeded_fill_host.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_ulonglong,
                                                 ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, ctypes.c_int]
        _host = lib
    return _host


def tensor_key(seed: int, name: str) -> int:
    raw = name.encode("utf-8")
    return int(_host_lib().coheryn_seeded_key(ctypes.c_ulonglong(int(seed) & (2 ** 64 - 1)), raw, len(raw)))


def seeded_tensor(seed: int, name: str, shape: Sequence[int], mean: float, deviation: float,
                  dtype: torch.dtype = torch.float32, device="cpu", first: int = 0) -> torch.Tensor:
    """The tensor ``name`` of the model made from ``seed``: element i holds value(first + i).
    On a CUDA device the values are made there by a kernel, on the CPU by the host runtime."""
    if dtype not in _KINDS:       # another storage type (float16 files): the float32 value, converted
        if not dtype.is_floating_point:
            raise ValueError(f"seeded tensors are floating-point, not {dtype}")
        return seeded_tensor(seed, name, shape, mean, deviation, torch.float32, device, first).to(dtype)
    device = torch.device(device)
    out = torch.empty(tuple(shape), dtype=dtype, device=device)
    n = out.numel()
    if n == 0:
        return out
    key = tensor_key(seed, name)
    if device.type == "cuda":
        from .. import ops
        ops.seeded_fill(out, key, first, float(mean), float(deviation))
    else:
        rc = _host_lib().coheryn_seeded_fill_host(
            ctypes.c_void_p(out.data_ptr()), _KINDS[dtype], ctypes.c_ulonglong(key), ctypes.c_ulonglong(first),
            ctypes.c_ulonglong(n), float(mean), float(deviation), min(32, os.cpu_count() or 1))
        if rc != 0:
            raise RuntimeError("the host runtime refused to fill a seeded tensor")
    return out
