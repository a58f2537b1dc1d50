"""Reading and writing the safetensors container (single file or indexed shards).

Layout: 8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the payload.  The checks follow the reference's reader
(crates/coheryn-engine/src/safetensors.rs:234-347): bounded header, duplicate keys
refused, only F32/F16/BF16 payloads (plus I32 for integer tables), byte ranges that
match ``shape x dtype`` exactly and cover the payload without holes or overlap;
``model.safetensors.index.json`` maps names to shard files whose names must be plain
basenames (safetensors.rs:432-547).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

MAX_HEADER_BYTES = 64 << 20

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate key {k!r} in safetensors header")
        out[k] = v
    return out


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int   # absolute file offset
    end: int
    path: str


def read_header(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: truncated before the header length")
        (n,) = struct.unpack("<Q", head)
        if n < 2 or n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} is out of range")
        raw = f.read(n)
    if len(raw) != n:
        raise SafetensorsError(f"{path}: truncated header")
    try:
        header = json.loads(raw.decode("utf-8"), object_pairs_hook=_no_duplicates)
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not an object")
    base = 8 + n
    payload = size - base
    entries: Dict[str, TensorEntry] = {}
    spans: List[Tuple[int, int, str]] = []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if not isinstance(info, dict):
            raise SafetensorsError(f"{path}: entry {name!r} is not an object")
        dt = info.get("dtype")
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r} "
                                   f"(supported: {', '.join(_DTYPES)})")
        shape = info.get("shape")
        offs = info.get("data_offsets")
        if (not isinstance(shape, list) or any(not isinstance(s, int) or s < 0 for s in shape)
                or not isinstance(offs, list) or len(offs) != 2
                or any(not isinstance(o, int) or o < 0 for o in offs)):
            raise SafetensorsError(f"{path}: tensor {name!r} has a malformed shape or offsets")
        count = 1
        for s in shape:
            count *= s
        b, e = offs
        if e < b or e > payload or e - b != count * _DTYPES[dt][1]:
            raise SafetensorsError(
                f"{path}: tensor {name!r} spans bytes {b}..{e}, which does not match "
                f"shape {shape} of {dt} inside a payload of {payload} bytes")
        entries[name] = TensorEntry(name, _DTYPES[dt][0], tuple(shape), base + b, base + e, path)
        spans.append((b, e, name))
    spans.sort()
    cursor = 0
    for b, e, name in spans:
        if b != cursor:
            raise SafetensorsError(f"{path}: payload has a hole or an overlap before {name!r}")
        cursor = e
    if cursor != payload:
        raise SafetensorsError(f"{path}: {payload - cursor} payload bytes belong to no tensor")
    return entries


def index_model_dir(model_dir: str) -> Dict[str, TensorEntry]:
    """All tensors of a model folder: ``model.safetensors`` or the shards named by
    ``model.safetensors.index.json``."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return read_header(single)
    if not os.path.isfile(index):
        raise SafetensorsError(f"{model_dir} holds neither model.safetensors nor "
                               "model.safetensors.index.json")
    with open(index, "rb") as f:
        obj = json.loads(f.read().decode("utf-8"), object_pairs_hook=_no_duplicates)
    weight_map = obj.get("weight_map") if isinstance(obj, dict) else None
    if not isinstance(weight_map, dict) or not weight_map:
        raise SafetensorsError(f"{index}: no weight_map")
    out: Dict[str, TensorEntry] = {}
    headers: Dict[str, Dict[str, TensorEntry]] = {}
    for name, shard in weight_map.items():
        if (not isinstance(shard, str) or os.path.basename(shard) != shard
                or shard in ("", ".", "..")):
            raise SafetensorsError(f"{index}: shard name {shard!r} is not a plain file name")
        if shard not in headers:
            headers[shard] = read_header(os.path.join(model_dir, shard))
        if name not in headers[shard]:
            raise SafetensorsError(f"{index}: {name!r} is not in shard {shard}")
        out[name] = headers[shard][name]
    for shard, h in headers.items():
        for name in h:
            if weight_map.get(name) != shard:
                raise SafetensorsError(f"{shard} holds {name!r}, which the index does not map to it")
    return out


class TensorReader:
    """Memory-maps the files of a set of entries and hands out tensors by name."""

    def __init__(self, entries: Dict[str, TensorEntry]):
        self.entries = entries
        self._maps: Dict[str, mmap.mmap] = {}

    def _map(self, path: str) -> mmap.mmap:
        m = self._maps.get(path)
        if m is None:
            with open(path, "rb") as f:
                m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[path] = m
        return m

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor holding a COPY of the stored values, in the stored dtype."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = self._map(e.path)
        flat = torch.frombuffer(bytearray(buf[e.begin:e.end]), dtype=torch.uint8)
        return flat.view(e.dtype).reshape(e.shape)

    def close(self) -> None:
        for m in self._maps.values():
            m.close()
        self._maps.clear()


def write_file(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Write tensors (in the given order) as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    cursor = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        if name in header:
            raise SafetensorsError(f"tensor {name!r} given twice")
        t = t.detach().contiguous().cpu()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [cursor, cursor + len(raw)]}
        cursor += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
