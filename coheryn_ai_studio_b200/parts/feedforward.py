"""Dense gated feed-forward: y = W_down (act(W_gate x) * (W_up x)), no biases; here act = silu (SwiGLU),
silu(g) = g / (1 + exp(-g)) in float32
(crates/coheryn-engine/src/inference.rs:516-540, crates/coheryn-engine/src/cpu.rs:74-78).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import FeedForward, Runtime, StepContext, register_feed_forward


class GatedMLP(FeedForward):
    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, activation: str):
        super().__init__(runtime)
        ops.gated_activation_code(activation)     # refuses, by name, an activation the epilogues lack
        self.activation = activation
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((I, H)), "up_proj.weight": TensorSpec((I, H)),
                "down_proj.weight": TensorSpec((H, I))}

    def bind(self, tensors):
        # One matrix product for gate and up, rows interleaved (2j = gate_j, 2j+1 = up_j) so
        # that the gated epilogue finds a pair in neighbouring output columns.
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        act = ops.gated_linear(x, self.w_gate_up, self.activation)
        return ops.linear(act, self.w_down, partial_ok=self.partial_output)


register_feed_forward("gated_mlp", GatedMLP)
