"""Interfaces of the parts a layer is assembled from, and the registries that map a
:class:`PartSpec` kind to a class.

A part is built from its parameters alone (``cls(**spec.params)`` plus the runtime's
dtype and device); it names the tensors it wants (:meth:`Part.tensor_specs`), receives
them (:meth:`Part.bind`) and runs on the device.  Roles:

* mixer         – ``forward(x, step, cache) -> y``; moves information between the tokens
                  of a request; says what cache it needs (:meth:`Mixer.cache_requirement`).
* feed_forward  – ``forward(x, step) -> y``; token-wise.
* norm          – ``forward(residual, delta, out_rows=None) -> normed``; adds ``delta`` to
                  the float32 residual stream in place and normalises.
* position      – owns what a mixer needs to encode positions (here: a rotation table).
* arrangement   – wires mixer, feed-forward and norms into a block.

New kinds are added with the ``register_*`` functions; nothing else has to change.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import PartSpec
from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision the parts run."""

    dtype: torch.dtype            # torch.float32 or torch.bfloat16: activations, matrices, cache
    device: torch.device


# ------------------------------------------------------------------ cache requirements
@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position (``window`` None) or of the last ``window``
    positions, kept in pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request, zeroed when the request is admitted."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What a mixer gets for one execution of its layer.

    Paged: ``k``/``v`` are ``[pages, kv heads, page_size, head_dim]`` views of the
    group's pool for this schedule entry; ``group`` indexes ``step.block_tables`` and
    ``step.slots``; ``writes`` is False when the entry reads another entry's cache.
    Fixed state: ``state`` is ``[slots, *shape]``; ``step.state_slots`` gives each
    request's slot."""

    kind: str                      # "paged" | "state"
    group: int = -1
    page_size: int = 0
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    writes: bool = True
    state: Optional[torch.Tensor] = None


@dataclass
class StepContext:
    """One batch of (request, its next tokens) as the device sees it.  Requests are
    numbered 0..B-1 in the order of the batch; their tokens are laid out one request
    after the other."""

    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor           # [T] int32
    positions: torch.Tensor           # [T] int32, absolute position of each token
    token_req: torch.Tensor           # [T] int32, batch index of each token's request
    cu_q: torch.Tensor                # [B+1] int32, token offsets of the requests
    kv_lens: torch.Tensor             # [B] int32, tokens of each request after this step
    block_tables: List[torch.Tensor]  # per cache group: [B, max_blocks] int32
    slots: List[torch.Tensor]         # per cache group: [T] int32 page*page_size+offset
    state_slots: torch.Tensor         # [B] int32
    q_lens: List[int] = field(default_factory=list)       # host copies
    kv_lens_host: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    # When few of the step's rows are wanted: the wanted rows as a step of their own (one row
    # per "request": one query at its position over the same pages) and their indices among the
    # step's tokens.  The LAST entry of the schedule then computes only these rows after it has
    # updated its cache for all of them (crates/coheryn-engine/src/inference.rs:481-485: a row
    # that needs no logits stops after the append in the last layer).  tail.num_tokens may be 0.
    tail: Optional["StepContext"] = None
    tail_rows: Optional[torch.Tensor] = None   # [R] int32
    # True (every ordinary step): what the cache holds at positions BEFORE a request's first token
    # of this step was written by earlier steps, so a kernel may read it ahead of the step's own
    # kernels.  False for the context of the wanted rows (``tail``): its one-token "requests" look
    # back on keys and values that this same step has just written.
    prior_positions_settled: bool = True
    # Scratch of parts/native_block.py: what the blocks of this step share once the first of them
    # has described the step to the library.
    native: Optional[object] = None


# ------------------------------------------------------------------------------- parts
class Part:
    # False if ``forward`` waits for the device (reads a result on the host) or launches work whose
    # shape depends on data: a model with such a part is never replayed from a CUDA graph.
    capturable = True

    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Local tensor name -> what is expected of it."""
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded tensors (same local names); may fuse or re-lay them."""


class Mixer(Part):
    # Set by the model when every norm takes partial sums: the part may then return its output
    # as a float32 stack [splits, T, H] whose sum is the output (see Norm.accepts_partial_sums).
    partial_output = False

    # True if the part implements forward_tail.
    supports_tail = False

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache) -> Optional[torch.Tensor]:
        """Update the cache (or state) for ALL rows of ``x`` as ``forward`` does, but return the
        output only for the rows ``step.tail_rows``, in that order (None when there are none);
        ``step.tail`` describes those rows as a step of their own."""
        raise NotImplementedError

    def cache_requirement(self):
        """PagedKV, FixedState or None."""
        return None

    def forward(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache]) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    partial_output = False   # as for Mixer

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    # True if ``delta`` may also be a float32 stack [splits, T, H] of partial sums, which the
    # norm adds in order before it adds them to the residual.
    accepts_partial_sums = False

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Position(Part):
    """What the stock attention asks of an encoding that turns pairs (i, i + rotary_dim / 2) of a
    head's first ``rotary_dim`` elements: the attribute ``rotary_dim`` and ``cos_sin()``, a float32
    device table [positions, rotary_dim / 2, 2] of (cos, sin).  A mixer of another kind may ask its
    position part for anything else."""


class Arrangement:
    """Wires the parts of one layer.  A subclass names its slots in ``SLOTS`` (slot name -> role:
    "mixer", "feed_forward" or "norm"; names in ``OPTIONAL`` may stay empty) and receives the
    built parts by slot name; each also becomes an attribute of that name (None when empty).
    ``forward`` takes and returns the pair (float32 residual stream, pending delta not yet added
    to it).  The model asks an arrangement only for what is below; it never names a slot."""

    SLOTS: Dict[str, str] = {}
    OPTIONAL: Tuple[str, ...] = ()

    def __init__(self, parts: Dict[str, Part]):
        unknown = sorted(set(parts) - set(self.SLOTS))
        missing = sorted(set(self.SLOTS) - set(parts) - set(self.OPTIONAL))
        if unknown or missing:
            raise ValueError(f"arrangement {type(self).__name__}: "
                             + (f"unknown slots {unknown} " if unknown else "")
                             + (f"missing slots {missing} " if missing else "")
                             + f"(slots: {sorted(self.SLOTS)})")
        self.slots = dict(parts)
        for name in self.SLOTS:
            setattr(self, name, parts.get(name))

    def parts(self) -> Dict[str, Part]:
        """Tensor-name component -> part (names follow the checkpoint)."""
        raise NotImplementedError

    def cache_owner(self) -> Optional[Part]:
        """The part whose ``cache_requirement`` decides what cache an execution of this layer
        gets (the first mixer by default), or None."""
        for name, role in self.SLOTS.items():
            if role == "mixer" and self.slots.get(name) is not None:
                return self.slots[name]
        return None

    def norms(self) -> List[Part]:
        return [self.slots[n] for n, role in self.SLOTS.items() if role == "norm" and n in self.slots]

    def producers(self) -> List[Part]:
        """The parts whose outputs go to a norm (mixers and feed-forwards)."""
        return [self.slots[n] for n, role in self.SLOTS.items() if role != "norm" and n in self.slots]

    def forward(self, residual, delta, step: StepContext, cache: Optional[LayerCache]):
        raise NotImplementedError

    # True if forward_tail may be called (the arrangement has one and its mixer can do it).
    supports_tail = False

    def forward_tail(self, residual, delta, step: StepContext, cache: Optional[LayerCache]):
        """As ``forward`` for the last entry of the schedule when ``step.tail`` is set: the
        returned pair holds only the rows ``step.tail_rows`` (or (None, None) without rows)."""
        raise NotImplementedError


MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
ARRANGEMENTS: Dict[str, type] = {}


def _register(table: Dict[str, type], role: str, kind: str, cls: type, replace: bool) -> None:
    if not kind:
        raise ValueError(f"a {role} needs a non-empty kind")
    if kind in table and not replace:
        raise ValueError(f"{role} kind {kind!r} is already registered")
    table[kind] = cls


def register_mixer(kind, cls, replace=False): _register(MIXERS, "mixer", kind, cls, replace)
def register_feed_forward(kind, cls, replace=False): _register(FEED_FORWARDS, "feed_forward", kind, cls, replace)
def register_norm(kind, cls, replace=False): _register(NORMS, "norm", kind, cls, replace)
def register_position(kind, cls, replace=False): _register(POSITIONS, "position", kind, cls, replace)
def register_arrangement(kind, cls, replace=False): _register(ARRANGEMENTS, "arrangement", kind, cls, replace)


def build_part(table: Dict[str, type], role: str, spec: PartSpec, runtime: Runtime, **extra):
    try:
        cls = table[spec.kind]
    except KeyError:
        raise ValueError(f"no {role} of kind {spec.kind!r} is registered "
                         f"(registered: {', '.join(sorted(table)) or 'none'})") from None
    return cls(runtime=runtime, **spec.params, **extra)
