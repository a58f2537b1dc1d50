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
        for ls in spec.layers:
            pos = None
            if ls.position is not None:
                key = repr(ls.position)
                if key not in self._positions:  # layers with the same encoding share its table
                    self._positions[key] = build_part(POSITIONS, "position", ls.position, runtime)
                pos = self._positions[key]
            extra = {"position": pos} if pos is not None else {}
            mixer = build_part(MIXERS, "mixer", ls.mixer, runtime, **extra)
            ff = build_part(FEED_FORWARDS, "feed_forward", ls.feed_forward, runtime)
            n1 = build_part(NORMS, "norm", ls.mixer_norm, runtime)
            n2 = build_part(NORMS, "norm", ls.feed_forward_norm, runtime)
            try:
                arr = ARRANGEMENTS[ls.arrangement]
            except KeyError:
                raise ValueError(f"no arrangement {ls.arrangement!r} is registered") from None
            self.layers.append(arr(mixer, ff, n1, n2))
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, runtime)
        # Outputs go from a layer to the NEXT norm (the following layer's, or the final one),
        # so partial sums may flow only if every norm of the model can add them.
        norms = [n for layer in self.layers for n in (layer.mixer_norm, layer.feed_forward_norm)] + [self.final_norm]
        if all(n.accepts_partial_sums for n in norms):
            for layer in self.layers:
                layer.mixer.partial_output = True
                layer.feed_forward.partial_output = True
        self.capturable = all(part.capturable for _, part in self._named_parts()) and all(
            p.capturable for p in self._positions.values())
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.status = None

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
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[f"{s.embedding_name}.weight"]
        for prefix, part in self._named_parts():
            local = {name: tensors[f"{prefix}.{name}"] for name in part.tensor_specs()
                     if f"{prefix}.{name}" in tensors}
            part.bind(local)
        self.head = tensors[f"{s.head_name}.weight"] if s.head_name is not None else self.embedding
        self.status = torch.zeros(1, dtype=torch.int32, device=self.runtime.device)

    # ------------------------------------------------------------------ cache needs
    def cache_requirements(self):
        """Per schedule entry: the mixer's requirement, or None when the entry reads an
        earlier entry's cache."""
        return [None if e.cache_from is not None else self.layers[e.layer].mixer.cache_requirement()
                for e in self.spec.schedule]

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepContext, caches: List[Optional[LayerCache]],
                logit_rows: torch.Tensor) -> torch.Tensor:
        """Run the step's tokens through the schedule; return float32 logits
        ``[len(logit_rows), vocab]`` of the rows asked for."""
        T, H = step.num_tokens, self.spec.hidden_size
        residual = torch.empty((T, H), dtype=torch.float32, device=self.runtime.device)
        ops.embed_gather(self.embedding, step.token_ids, residual, self.status)
        delta = None
        last = len(self.spec.schedule) - 1
        tailed = False
        for i, (entry, cache) in enumerate(zip(self.spec.schedule, caches)):
            layer = self.layers[entry.layer]
            if i == last and step.tail is not None and layer.supports_tail:
                residual, delta = layer.forward_tail(residual, delta, step, cache)
                tailed = True
            else:
                residual, delta = layer.forward(residual, delta, step, cache)
        R = logit_rows.numel()
        if R == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.runtime.device)
        h = self.final_norm.forward(residual, delta, rows=None if tailed else logit_rows)
        return ops.linear(h, self.head, out_dtype=torch.float32)
