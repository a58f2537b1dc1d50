"""Arrangements: how a layer's mixer, feed-forward and norms are wired.

``prenorm_residual`` is the layout of crates/coheryn-engine/src/inference.rs:440-540:
x += mixer(norm(x)); x += feed_forward(norm(x)).  The residual stream is float32; each
sub-layer's output is handed on as a pending ``delta`` that the NEXT norm adds to the
stream while it normalises, so the sum and the norm cost one pass over the row.
"""
from __future__ import annotations

from typing import Dict

from .. import ops
from .base import Arrangement, Part, register_arrangement
from .native_block import NativeBlock


class PreNormResidual(Arrangement):
    SLOTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def parts(self) -> Dict[str, Part]:
        return {"input_layernorm": self.mixer_norm, "self_attn": self.mixer,
                "post_attention_layernorm": self.feed_forward_norm, "mlp": self.feed_forward}

    _native = None     # None: not looked at yet; False: not made of the built-in parts

    def _native_block(self):
        nb = self._native
        if nb is None or (nb is not False and not nb.current(self)):
            nb = self._native = NativeBlock.build(self) or False
        return nb

    def forward(self, residual, delta, step, cache):
        if ops.NATIVE_BLOCK:
            nb = self._native_block()
            if nb:
                out = nb.run(residual, delta, step, cache)   # the whole block from one call into the library
                if out is not None:
                    return residual, out
        mixed = self.mixer.forward(self.mixer_norm.forward(residual, delta), step, cache)
        out = self.feed_forward.forward(self.feed_forward_norm.forward(residual, mixed), step)
        return residual, out

    @property
    def supports_tail(self):
        return self.mixer.supports_tail

    def forward_tail(self, residual, delta, step, cache):
        mixed = self.mixer.forward_tail(self.mixer_norm.forward(residual, delta), step, cache)
        if mixed is None:
            return None, None
        kept = ops.gather_rows(residual, step.tail_rows)
        out = self.feed_forward.forward(self.feed_forward_norm.forward(kept, mixed), step.tail)
        return kept, out


register_arrangement("prenorm_residual", PreNormResidual)
