"""RMSNorm fused with the residual add.

y = (x * (1 / sqrt(mean(x^2) + eps))) * w in float32, the order of operations of
crates/coheryn-engine/src/cpu.rs:49-57 (which sums the squares in float64; here the sum
is a float32 tree of fixed shape).  The weight has no bias and no "+1".
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Norm, Runtime, register_norm


class RMSNorm(Norm):
    accepts_partial_sums = True

    def __init__(self, runtime: Runtime, size: int, eps: float):
        super().__init__(runtime)
        self.size, self.eps = int(size), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), role="vector", init="norm")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, residual, delta, rows=None):
        """residual += delta (when given and no ``rows``); returns the normalised rows in
        the compute dtype.  With ``rows`` only those rows are produced."""
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.runtime.dtype, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows)
        return out


register_norm("rmsnorm", RMSNorm)
