"""Grouped-query causal attention over cache pages.

Formulas as the reference runs them (crates/coheryn-engine/src/inference.rs:450-508,
crates/coheryn-engine/src/cpu.rs:133-210): q, k, v = W x + b; rotate q and k by
position; append k, v to the cache; for head h of group g = h // (heads // kv_heads),
s_t = (q_h . K[t, g]) * scale over the cached positions t <= p, softmax in float32,
o_h = sum_t P_t V[t, g]; y = W_o o (+ b_o).  A ``window`` keeps only the last
``window`` positions (t > p - window).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import LayerCache, Mixer, PagedKV, Position, Runtime, StepContext, register_mixer


class Attention(Mixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qkv_bias: bool, o_bias: bool, window: Optional[int], scale: float,
                 position: Optional[Position] = None):
        super().__init__(runtime)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if window is not None and window < 1:
            raise ValueError("an attention window must hold at least one position")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.qkv_bias, self.o_bias = head_dim, bool(qkv_bias), bool(o_bias)
        self.window, self.scale, self.position = window, float(scale), position
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H = self.hidden_size
        specs = {
            "q_proj.weight": TensorSpec((self.q_size, H)),
            "k_proj.weight": TensorSpec((self.kv_size, H)),
            "v_proj.weight": TensorSpec((self.kv_size, H)),
            "o_proj.weight": TensorSpec((H, self.q_size)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((self.q_size,), role="vector", init="bias")
            specs["k_proj.bias"] = TensorSpec((self.kv_size,), role="vector", init="bias")
            specs["v_proj.bias"] = TensorSpec((self.kv_size,), role="vector", init="bias")
        if self.o_bias:
            specs["o_proj.bias"] = TensorSpec((H,), role="vector", init="bias")
        return specs

    def bind(self, tensors):
        # One matrix product for q, k and v: rows of the three matrices stacked.
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        if self.qkv_bias:
            biases = [tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]
            dt = torch.float32 if any(b.dtype == torch.float32 for b in biases) else biases[0].dtype
            self.b_qkv = torch.cat([b.to(dt) for b in biases]).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors.get("o_proj.bias")

    def _rotated_queries(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        """q, k, v of every row; k and v (rotated k) written to the cache; returns the rotated q
        [T, heads * head size] (possibly a column slice of a wider buffer).  Three ways to the same
        values: few rows (decoding) rotate and write in the product's own epilogue; a product whose K
        the many-rows kernel splits leaves the addition of its slices to the rotation kernel; otherwise
        the product, then the rotation kernel."""
        rot = self.position.rotary_dim if self.position is not None else 0
        cos_sin = self.position.cos_sin() if self.position is not None else None
        slots = step.slots[cache.group]
        if self.position is not None and ops.qkv_rope_ok(x, self.w_qkv, cache.k, rot, self.head_dim):
            return ops.qkv_rope_small(x, self.w_qkv, self.b_qkv, step.positions, cos_sin, slots, cache.k, cache.v,
                                      self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size)
        count = ops.qkv_parts_count(x, self.w_qkv, cache.k, rot, self.head_dim) if self.position is not None else 0
        if count > 1:
            return ops.qkv_rope_parts(x, self.w_qkv, self.b_qkv, step.positions, cos_sin, slots, cache.k, cache.v,
                                      self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, count)
        qkv = ops.linear(x, self.w_qkv, self.b_qkv)
        ops.rope_kv_write(qkv, step.positions, cos_sin, slots, cache.k, cache.v, self.num_heads, self.num_kv_heads,
                          self.head_dim, rot, cache.page_size)
        return qkv[:, :self.q_size]

    def _queries_only(self, x: torch.Tensor, positions: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        """For an execution that reads keys and values another one wrote: only q is made and rotated."""
        b = self.b_qkv[:self.q_size] if self.b_qkv is not None else None
        q = ops.linear(x, self.w_qkv[:self.q_size], b)
        rot = self.position.rotary_dim if self.position is not None else 0
        cos_sin = self.position.cos_sin() if self.position is not None else None
        ops.rope_kv_write(q, positions, cos_sin, None, None, None, self.num_heads, 0, self.head_dim, rot, cache.page_size)
        return q

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        self._check(cache)
        q = self._rotated_queries(x, step, cache) if cache.writes else self._queries_only(x, step.positions, cache)
        return self._attend_q(q, step, cache)

    supports_tail = True

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> Optional[torch.Tensor]:
        """Keys and values of every row go to the cache; only the wanted rows attend."""
        self._check(cache)
        rows, tail = step.tail_rows, step.tail
        if not cache.writes:   # nothing to write: the wanted rows alone make their queries
            if not tail.num_tokens:
                return None
            return self._attend_q(self._queries_only(ops.gather_rows(x, rows), tail.positions, cache), tail, cache)
        q = self._rotated_queries(x, step, cache)
        if not tail.num_tokens:
            return None
        return self._attend_q(ops.gather_rows(q, rows), tail, cache)

    @staticmethod
    def _check(cache) -> None:
        if cache is None or cache.kind != "paged":
            raise ValueError("attention needs a paged key/value cache")

    def _attend_q(self, q: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        """Attention of rotated queries over the cache, then the output projection."""
        if self.partial_output and ops.attention_oproj_ok(q, self.w_o, step, self.num_heads, self.num_kv_heads, self.head_dim):
            # a small decode batch: the splits of the attention are merged inside the projection's kernel,
            # and the heads' contributions go to the next norm as partial sums
            return ops.attention_oproj(q, cache.k, cache.v, step, cache.group, self.num_heads, self.num_kv_heads,
                                       self.head_dim, cache.page_size, self.window, self.scale, self.w_o, self.b_o)
        o = torch.empty((q.shape[0], self.q_size), dtype=q.dtype, device=q.device)
        ops.attention(q, o, cache.k, cache.v, step, cache.group, self.num_heads, self.num_kv_heads, self.head_dim,
                      cache.page_size, self.window, self.scale)
        return ops.linear(o, self.w_o, self.b_o, partial_ok=self.partial_output)


register_mixer("attention", Attention)
