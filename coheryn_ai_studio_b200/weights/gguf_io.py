"""GGUF (version 3) files with unquantized tensors: metadata and a tensor index.

The container as the reference reads it (crates/coheryn-engine/src/gguf.rs:20-140): magic
"GGUF", version, tensor count, key/value count, the key/value pairs, the tensor infos
(name, dimensions innermost first, type, offset into the data section), then the data
section at the next multiple of ``general.alignment`` (32 when absent).  Only F32 (type 0),
F16 (1) and BF16 (30) tensors are taken; a packed type is an error that names the tensor,
as crates/coheryn-engine/src/compat.rs:234-244 does.  GGML lists a matrix's dimensions as
[in, out] with ``in`` contiguous, which is byte for byte a row-major [out, in] matrix, so a
tensor's shape here is its dimensions reversed and no data moves.

``write_gguf`` writes such a file (tests and the random-weights mode).
"""
from __future__ import annotations

import os
import struct
from typing import Any, Dict, Iterable, List, Tuple

import torch

from .safetensors_io import TensorEntry

MAGIC = b"GGUF"
MAX_METADATA_BYTES = 256 << 20
MAX_STRING = 1 << 24
MAX_DIMS = 4

_TENSOR_TYPES = {0: (torch.float32, 4), 1: (torch.float16, 2), 30: (torch.bfloat16, 2)}
_TYPE_IDS = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY = 8, 9


class GgufError(ValueError):
    pass


class _Cursor:
    def __init__(self, f, limit: int):
        self.f, self.limit = f, limit

    def take(self, n: int) -> bytes:
        if n < 0 or self.f.tell() + n > self.limit:
            raise GgufError("the GGUF header runs past the end of the file")
        b = self.f.read(n)
        if len(b) != n:
            raise GgufError("the GGUF file is truncated")
        return b

    def scalar(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.scalar("<Q")
        if n > MAX_STRING:
            raise GgufError(f"a GGUF string of {n} bytes is refused")
        try:
            return self.take(n).decode("utf-8")
        except UnicodeDecodeError:
            raise GgufError("a GGUF string is not UTF-8") from None

    def value(self, vtype: int, depth: int = 0):
        if vtype in _SCALARS:
            return self.scalar(_SCALARS[vtype])
        if vtype == T_STRING:
            return self.string()
        if vtype == T_ARRAY:
            if depth:
                raise GgufError("nested GGUF arrays are refused")
            etype, count = self.scalar("<I"), self.scalar("<Q")
            if etype in _SCALARS:      # read in one piece: token tables hold 10^5 entries
                fmt = _SCALARS[etype]
                size = struct.calcsize(fmt)
                raw = self.take(size * count)
                return list(struct.unpack(f"<{count}{fmt[1]}", raw))
            return [self.value(etype, 1) for _ in range(count)]
        raise GgufError(f"unknown GGUF value type {vtype}")


def read_gguf(path: str) -> Tuple[Dict[str, Any], Dict[str, TensorEntry]]:
    """(metadata, tensor index by GGUF name).  Shapes are row-major (dimensions reversed)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        c = _Cursor(f, min(size, MAX_METADATA_BYTES))
        if c.take(4) != MAGIC:
            raise GgufError(f"{path} is not a GGUF file")
        version = c.scalar("<I")
        if version != 3:
            raise GgufError(f"GGUF version {version} is not read (3 is)")
        n_tensors, n_kv = c.scalar("<Q"), c.scalar("<Q")
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = c.string()
            if key in meta:
                raise GgufError(f"duplicate GGUF key {key!r}")
            meta[key] = c.value(c.scalar("<I"))
        infos: List[Tuple[str, Tuple[int, ...], int, int]] = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.scalar("<I")
            if not 1 <= nd <= MAX_DIMS:
                raise GgufError(f"tensor {name} has {nd} dimensions")
            dims = tuple(c.scalar("<Q") for _ in range(nd))
            infos.append((name, dims, c.scalar("<I"), c.scalar("<Q")))
        header_end = f.tell()
    align = meta.get("general.alignment", 32)
    if not isinstance(align, int) or align <= 0 or align & (align - 1):
        raise GgufError(f"general.alignment {align!r} is not a power of two")
    data0 = -(-header_end // align) * align
    entries: Dict[str, TensorEntry] = {}
    spans = []
    for name, dims, ttype, offset in infos:
        if name in entries:
            raise GgufError(f"duplicate tensor {name!r}")
        if ttype not in _TENSOR_TYPES:
            raise GgufError(f"tensor {name} has GGML type {ttype}: only F32, F16 and BF16 tensors are read "
                            "(packed types are not implemented)")
        dtype, item = _TENSOR_TYPES[ttype]
        count = 1
        for d in dims:
            count *= d
        begin = data0 + offset
        end = begin + count * item
        if offset % align or end > size:
            raise GgufError(f"tensor {name} lies outside the file or off its alignment")
        spans.append((begin, end, name))
        entries[name] = TensorEntry(name, dtype, tuple(reversed(dims)), begin, end, path)
    spans.sort()
    for (b0, e0, n0), (b1, _, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise GgufError(f"tensors {n0} and {n1} overlap")
    return meta, entries


def _put_string(out: bytearray, s: str) -> None:
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _put_value(out: bytearray, v) -> None:
    if isinstance(v, bool):
        out += struct.pack("<I?", 7, v)
    elif isinstance(v, int):
        out += struct.pack("<II", 4, v) if 0 <= v < 1 << 32 else struct.pack("<Iq", 11, v)
    elif isinstance(v, float):
        out += struct.pack("<If", 6, v)
    elif isinstance(v, str):
        out += struct.pack("<I", T_STRING)
        _put_string(out, v)
    elif isinstance(v, (list, tuple)):
        out += struct.pack("<I", T_ARRAY)
        if all(isinstance(x, str) for x in v):
            out += struct.pack("<IQ", T_STRING, len(v))
            for x in v:
                _put_string(out, x)
        elif all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            out += struct.pack("<IQ", 5, len(v)) + struct.pack(f"<{len(v)}i", *v)
        else:
            raise GgufError("only arrays of strings or of integers are written")
    else:
        raise GgufError(f"a {type(v).__name__} is not written to GGUF metadata")


def write_gguf(path: str, metadata: Dict[str, Any], tensors: Iterable[Tuple[str, torch.Tensor]],
               alignment: int = 32) -> None:
    """Write metadata and F32 / F16 / BF16 tensors (given row-major, stored with GGML's
    reversed dimension order)."""
    tensors = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    head = bytearray(MAGIC + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for k, v in metadata.items():
        _put_string(head, k)
        _put_value(head, v)
    offset = 0
    offsets = []
    for name, t in tensors:
        if t.dtype not in _TYPE_IDS:
            raise GgufError(f"tensor {name}: dtype {t.dtype} is not written")
        _put_string(head, name)
        head += struct.pack("<I", t.dim()) + struct.pack(f"<{t.dim()}Q", *reversed(t.shape))
        head += struct.pack("<IQ", _TYPE_IDS[t.dtype], offset)
        offsets.append(offset)
        offset = -(-(offset + t.numel() * t.element_size()) // alignment) * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (-len(head) % alignment))
        data0 = f.tell()
        for (name, t), off in zip(tensors, offsets):
            f.seek(data0 + off)
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
        f.truncate(max(f.tell(), data0 + offset))
