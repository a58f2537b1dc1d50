"""Architecture-neutral description of a decoder: which parts make up each layer,
with what parameters, and in what order layers run.

A model configuration (for example :class:`Qwen2Config`) is translated into a
:class:`ModelSpec` by the function registered for its architecture name.  Everything
below the registry (parts, cache manager, step function, scheduler) sees only the
:class:`ModelSpec`; no part knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` selects the class from the part registry of its
    role (mixer, feed_forward, norm, position); ``params`` are its constructor
    arguments (sizes and constants, never read from a global)."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A layer = an arrangement (how the parts are wired, e.g. pre-norm residual) over the parts
    that fill its slots.  ``parts`` maps a slot name of the arrangement (for the pre-norm block:
    ``mixer``, ``feed_forward``, ``mixer_norm``, ``feed_forward_norm``) to the part that fills it;
    which slots exist, which may stay empty and what role each has is the arrangement's business,
    so a block without a feed-forward, with four norms or with two mixers is another arrangement
    and nothing else.  ``position`` is handed to the layer's mixers.  ``prefix`` is the
    tensor-name prefix of the layer's weights (``model.layers.3``)."""

    prefix: str
    arrangement: str
    parts: Mapping[str, PartSpec]
    position: Optional[PartSpec] = None


def prenorm_layer(prefix: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                  feed_forward_norm: PartSpec, position: Optional[PartSpec] = None) -> LayerSpec:
    """The usual block: x += mixer(norm(x)); x += feed_forward(norm(x))."""
    return LayerSpec(prefix, "prenorm_residual",
                     {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": mixer_norm,
                      "feed_forward_norm": feed_forward_norm}, position)


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  The schedule is a list of these: a layer may be
    named twice (it then runs twice with the same weights, each run with a cache of
    its own), and ``cache_from`` lets an entry read the cache that an EARLIER entry
    of the schedule wrote instead of owning one."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    final_norm_name: str
    head_name: Optional[str]  # None: logits use the embedding table (tied)
    # Options that some architectures have and this one leaves at "none": the embedding rows are
    # multiplied by ``embedding_scale``; the logits are multiplied by ``logit_scale`` and a bias
    # ``head_bias_name`` (full tensor name, [vocab]) is added to them.
    embedding_scale: Optional[float] = None
    logit_scale: Optional[float] = None
    head_bias_name: Optional[str] = None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the schedule names no layer")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                        "which is not an earlier entry")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                        "which owns no cache itself")
