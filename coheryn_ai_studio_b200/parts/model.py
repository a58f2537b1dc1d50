"""The decoder as data: an embedding, layers built from a ModelSpec, a schedule that says
in which order (and how often, and with whose cache) they run, a final norm and the
output head.  It knows no architecture by name.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..config.spec import ModelSpec
from ..weights.spec import TensorSpec
from . import attention, block, feedforward, norm, position  # noqa: F401  (register the stock parts)
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, LayerCache, Part,
                   Runtime, StepContext, build_part)


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec, self.runtime = spec, runtime
        self._positions: Dict[str, Part] = {}
        self.layers = []
        tables = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}
        for ls in spec.layers:
            pos = None
            if ls.position is not None:
                key = repr(ls.position)
                if key not in self._positions:  # layers with the same encoding share its table
                    self._positions[key] = build_part(POSITIONS, "position", ls.position, runtime)
                pos = self._positions[key]
            try:
                arr = ARRANGEMENTS[ls.arrangement]
            except KeyError:
                raise ValueError(f"no arrangement {ls.arrangement!r} is registered") from None
            built = {}
            for slot, part_spec in ls.parts.items():
                role = arr.SLOTS.get(slot)
                if role is None:
                    raise ValueError(f"layer {ls.prefix}: arrangement {ls.arrangement!r} has no slot {slot!r} "
                                     f"(slots: {sorted(arr.SLOTS)})")
                extra = {"position": pos} if role == "mixer" and pos is not None else {}
                built[slot] = build_part(tables[role], role, part_spec, runtime, **extra)
            self.layers.append(arr(built))
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, runtime)
        # Outputs go from a layer to the NEXT norm (the following layer's, or the final one),
        # so partial sums may flow only if every norm of the model can add them.
        norms = [n for layer in self.layers for n in layer.norms()] + [self.final_norm]
        if all(n.accepts_partial_sums for n in norms):
            for layer in self.layers:
                for part in layer.producers():
                    part.partial_output = True
        self.capturable = all(part.capturable for _, part in self._named_parts()) and all(
            p.capturable for p in self._positions.values())
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.head_bias: Optional[torch.Tensor] = None
        self.status = None
        # Called with (schedule entry, float32 [T, H] output of that entry) when set: the layer
        # outputs of a trace (crates/coheryn-engine/src/inference.rs:541-543).  Off in serving.
        self.layer_observer = None

    # ------------------------------------------------------------------ tensors
    def _named_parts(self) -> List[Tuple[str, Part]]:
        out = []
        for ls, layer in zip(self.spec.layers, self.layers):
            for comp, part in layer.parts().items():
                out.append((f"{ls.prefix}.{comp}", part))
        out.append((self.spec.final_norm_name, self.final_norm))
        return out

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Every tensor the checkpoint must hold, by its full name."""
        s = self.spec
        specs = {f"{s.embedding_name}.weight": TensorSpec((s.vocab_size, s.hidden_size))}
        for prefix, part in self._named_parts():
            for local, ts in part.tensor_specs().items():
                specs[f"{prefix}.{local}"] = ts
        if s.head_name is not None:
            specs[f"{s.head_name}.weight"] = TensorSpec((s.vocab_size, s.hidden_size))
        if s.head_bias_name is not None:
            specs[s.head_bias_name] = TensorSpec((s.vocab_size,), role="vector", init="bias")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[f"{s.embedding_name}.weight"]
        for prefix, part in self._named_parts():
            local = {name: tensors[f"{prefix}.{name}"] for name in part.tensor_specs()
                     if f"{prefix}.{name}" in tensors}
            part.bind(local)
        self.head = tensors[f"{s.head_name}.weight"] if s.head_name is not None else self.embedding
        self.head_bias = tensors[s.head_bias_name] if s.head_bias_name is not None else None
        self.status = torch.zeros(1, dtype=torch.int32, device=self.runtime.device)

    # ------------------------------------------------------------------ cache needs
    def cache_requirements(self):
        """Per schedule entry: the mixer's requirement, or None when the entry reads an
        earlier entry's cache."""
        def need(entry):
            owner = self.layers[entry.layer].cache_owner()
            return owner.cache_requirement() if owner is not None and entry.cache_from is None else None
        return [need(e) for e in self.spec.schedule]

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepContext, caches: List[Optional[LayerCache]],
                logit_rows: torch.Tensor) -> torch.Tensor:
        """Run the step's tokens through the schedule; return float32 logits
        ``[len(logit_rows), vocab]`` of the rows asked for."""
        T, H = step.num_tokens, self.spec.hidden_size
        step.native = None      # a step object may be run again (warm-up, then capture): on another stream
        residual = torch.empty((T, H), dtype=torch.float32, device=self.runtime.device)
        ops.embed_gather(self.embedding, step.token_ids, residual, self.status, scale=self.spec.embedding_scale)
        delta = None
        last = len(self.spec.schedule) - 1
        tailed = False
        for i, (entry, cache) in enumerate(zip(self.spec.schedule, caches)):
            layer = self.layers[entry.layer]
            if i == last and step.tail is not None and layer.supports_tail and self.layer_observer is None:
                residual, delta = layer.forward_tail(residual, delta, step, cache)
                tailed = True
            else:
                residual, delta = layer.forward(residual, delta, step, cache)
            if self.layer_observer is not None:
                out = residual if delta is None else residual + (delta.sum(0) if delta.dim() == 3 else delta.float())
                self.layer_observer(i, out)
        R = logit_rows.numel()
        if R == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.runtime.device)
        h = self.final_norm.forward(residual, delta, rows=None if tailed else logit_rows)
        logits = ops.linear(h, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale is not None or self.head_bias is not None:
            ops.scale_add_bias(logits, self.spec.logit_scale, self.head_bias)
        return logits
