"""What a part says about each tensor it wants from the checkpoint."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class TensorSpec:
    """``role`` decides the dtype the tensor is kept in:

    * ``matrix``  – an operand of a matrix product or the embedding table: kept in the
      compute dtype (bfloat16 or float32);
    * ``vector``  – norm weights, biases and other small tables: a tensor stored in
      32-bit stays 32-bit, a 16-bit one is kept in the compute dtype;
    * ``int_table`` – integer tables, kept as int32.

    ``init`` names how the random-weights mode fills it: ``normal`` (matrix_std),
    ``bias`` (bias_std), ``norm`` (1 + norm_jitter * N(0,1)), ``zeros``.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False
