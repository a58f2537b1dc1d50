"""A pre-norm block of the built-in parts enqueued by one call into the library.

``PreNormResidual.forward`` runs its four parts one after the other; each is a few calls into the
library with checks and allocations between them, about 150 us of host time per layer.  Steps that
are replayed from a CUDA graph do not pay that, every other step does (prompt portions, mixed
batches), and at small layer sizes it bounds them.  When the block is made of exactly the built-in
attention, gated feed-forward and RMSNorm parts in bfloat16, ``NativeBlock`` hands the whole block to
``coheryn_prenorm_block_bf16`` (csrc/block_runner.cu), which makes the same choices of kernels from
the same thresholds (they are read from ``ops`` at every step) and calls the same entry points.
Anything else (another part, a cache that is only read, a shape the library's sequence does not
cover) takes the parts' own path: ``run`` returns None.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .. import ops

P = c_void_p


class CoBlockLayer(ctypes.Structure):
    _fields_ = [(n, P) for n in ("norm1_w", "norm2_w", "w_qkv", "b_qkv", "w_o", "b_o", "w_gate_up", "w_down", "cos_sin",
                                 "attention", "attention_oproj", "attn_scratch_floats")] + \
               [(n, c_float) for n in ("eps1", "eps2", "scale")] + \
               [(n, c_int) for n in ("norm1_wdtype", "norm2_wdtype", "b_qkv_dtype", "b_o_dtype", "H", "nh", "nkv", "hd", "I",
                                     "rot", "window", "gated_code", "mixer_partial", "ff_partial")]


class CoBlockStep(ctypes.Structure):
    _fields_ = [(n, P) for n in ("positions", "cu_q", "kv_lens", "tc_status", "stream")] + \
               [(n, c_int) for n in ("T", "B", "min_q_len", "max_q_len", "max_kv_len", "settled")]


class CoBlockTuning(ctypes.Structure):
    _fields_ = [(n, c_long) for n in ("small_weight_elements", "few_large_weight", "attn_oproj_merge_bytes")] + \
               [(n, c_int) for n in ("few_m", "few_defer_m", "few_head_m", "small_m", "small_m_short", "defer_min_k",
                                     "defer_min_k_wide", "qkv_rope_m", "qkv_parts_m", "qkv_parts_few_from", "attn_oproj_m")]


class CoBlockPlan(ctypes.Structure):
    _fields_ = [("scratch_bytes", c_long), ("out_kind", c_int), ("out_splits", c_int)] + \
               [(n, c_int) for n in ("qkv_route", "qkv_parts", "qkv_linear", "merged", "o_route", "gate_route", "down_route")]


UNSUPPORTED, ATTENTION_FAILED = 3, 2

# Blocks enqueued through the library since the module was loaded (tests look at it).
runs = 0


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return t.data_ptr() if t is not None else None


def _i32(t) -> bool:
    return t is not None and t.dtype == torch.int32 and t.is_contiguous() and t.is_cuda


# The blocks' temporaries: one area per device, grown when a step needs more, never given back
# (a captured graph may name an area that has been outgrown, so those stay alive too).  The blocks of
# a device run in stream order on one stream, as the few-rows product's workspace already requires.
# An area per step would be simpler, but areas of changing size (portions of changing length) sent
# the allocator to the driver: the 7B serving run was 2 % slower with them.
_scratch = {}
_retired = []


def _scratch_for(device, nbytes: int):
    got = _scratch.get(device)
    if got is None or got[1] < nbytes:
        if got is not None:
            _retired.append(got[2])
        size = max(nbytes + (nbytes >> 2), 64 << 20)
        t = torch.empty(size, dtype=torch.uint8, device=device)
        got = _scratch[device] = (t.data_ptr(), size, t)
    return got


_entry = None


def _entry_point():
    """The library's function with its argument types declared once (plain integers then pass as
    pointers and sizes without a wrapper object each)."""
    global _entry
    if _entry is None:
        fn = ops.core().coheryn_prenorm_block_bf16
        fn.argtypes = [P, P, P, P, P, c_int, c_int, P, c_int, P, P, P, c_int, c_int, P, c_int, c_int, P, c_long, c_int, P]
        fn.restype = c_int
        _entry = fn
    return _entry


class StepNative:
    """What every block of one step shares: the step's description and thresholds as the library
    reads them, the pointers of each cache group's tables, and per kind of layer the plan (kind of
    output, scratch area)."""

    def __init__(self, step):
        self.ok = False
        q_lens = step.q_lens
        if (not q_lens or not step.max_kv_len or len(q_lens) != step.num_requests or step.num_tokens <= 0
                or not (_i32(step.positions) and _i32(step.cu_q) and _i32(step.kv_lens))):
            return
        device = step.positions.device
        self.step = CoBlockStep(step.positions.data_ptr(), step.cu_q.data_ptr(), step.kv_lens.data_ptr(),
                                ops.tc_status(device).data_ptr(), ops._stream().value or 0, step.num_tokens, len(q_lens),
                                min(q_lens), max(q_lens), step.max_kv_len, 1 if step.prior_positions_settled else 0)
        self.tuning = CoBlockTuning(ops.SMALL_WEIGHT_ELEMENTS, ops.FEW_LARGE_WEIGHT, ops.ATTN_OPROJ_MERGE_BYTES, ops.FEW_M,
                                    ops.FEW_DEFER_M, ops.FEW_HEAD_M, ops.SMALL_M, ops.SMALL_M_SHORT, ops.DEFER_MIN_K,
                                    ops.DEFER_MIN_K_WIDE, ops.QKV_ROPE_M, ops.QKV_PARTS_M, ops.QKV_PARTS_FEW_FROM,
                                    ops.ATTN_OPROJ_M)
        self.step_ref, self.tuning_ref = ctypes.addressof(self.step), ctypes.addressof(self.tuning)
        self.groups = {}
        self.plans = {}
        self.device = device
        self.ok = True

    def group(self, step, g: int):
        got = self.groups.get(g)
        if got is None:
            bt, slots = step.block_tables[g], step.slots[g]
            got = (bt.data_ptr(), bt.shape[1], slots.data_ptr()) if _i32(bt) and _i32(slots) and bt.dim() == 2 else False
            self.groups[g] = got
        return got


class NativeBlock:
    def __init__(self, layer: CoBlockLayer, key, keep):
        self.layer, self.key, self.keep = layer, key, keep
        self.layer_ref = ctypes.addressof(layer)
        self.plan = CoBlockPlan()
        self.plan_ref = ctypes.addressof(self.plan)

    @classmethod
    def build(cls, arrangement) -> Optional["NativeBlock"]:
        """The description of ``arrangement`` for the library, or None if it is not made of the
        built-in parts in bfloat16 (exact classes: a subclass may compute something else)."""
        from .attention import Attention
        from .feedforward import GatedMLP
        from .norm import RMSNorm
        m, f = arrangement.mixer, arrangement.feed_forward
        n1, n2 = arrangement.mixer_norm, arrangement.feed_forward_norm
        if not (type(m) is Attention and type(f) is GatedMLP and type(n1) is RMSNorm and type(n2) is RMSNorm):
            return None
        if m.runtime.dtype != torch.bfloat16 or m.position is None or m.w_qkv is None or f.w_gate_up is None:
            return None
        cos_sin, rot = m.position.cos_sin(), int(m.position.rotary_dim)
        H, I = m.hidden_size, f.intermediate_size
        weights = (m.w_qkv, m.w_o, f.w_gate_up, f.w_down)
        shapes = (((m.num_heads + 2 * m.num_kv_heads) * m.head_dim, H), (H, m.q_size), (2 * I, H), (H, I))
        if any(w.dtype != torch.bfloat16 or not w.is_contiguous() or not w.is_cuda or tuple(w.shape) != s
               or w.data_ptr() % 16 for w, s in zip(weights, shapes)):
            return None
        if not (cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and tuple(cos_sin.shape[1:]) == (rot // 2, 2)
                and 0 < rot <= m.head_dim and rot % 2 == 0):
            return None
        vectors = (n1.weight, n2.weight, m.b_qkv, m.b_o)
        if any(v is not None and (v.dtype not in (torch.float32, torch.bfloat16) or not v.is_contiguous()) for v in vectors):
            return None
        if n1.size != H or n2.size != H or f.hidden_size != H or n1.weight.shape != (H,) or n2.weight.shape != (H,):
            return None
        try:
            gated = ops.gated_activation_code(f.activation)
            lib = ops.attention_lib(m.head_dim)
        except Exception:
            return None
        fn = lambda f_: ctypes.cast(f_, c_void_p).value
        code = lambda t: ops._code(t) if t is not None else ops.F32
        layer = CoBlockLayer(_ptr(n1.weight), _ptr(n2.weight), _ptr(m.w_qkv), _ptr(m.b_qkv), _ptr(m.w_o), _ptr(m.b_o),
                             _ptr(f.w_gate_up), _ptr(f.w_down), _ptr(cos_sin), fn(lib.coheryn_attention_bf16),
                             fn(lib.coheryn_attention_oproj_bf16), fn(lib.coheryn_attn_scratch_floats), n1.eps, n2.eps,
                             m.scale, code(n1.weight), code(n2.weight), code(m.b_qkv), code(m.b_o), H, m.num_heads,
                             m.num_kv_heads, m.head_dim, I, rot, int(m.window or 0), gated,
                             1 if m.partial_output else 0, 1 if f.partial_output else 0)
        key = (H, m.num_heads, m.num_kv_heads, m.head_dim, I, rot, int(m.window or 0), gated, bool(m.partial_output),
               bool(f.partial_output), code(m.b_qkv) if m.b_qkv is not None else -1, code(m.b_o) if m.b_o is not None else -1)
        return cls(layer, key, (weights, vectors, cos_sin, lib))

    def current(self, arrangement) -> bool:
        """False once a part's tensors were bound anew (the description holds their addresses)."""
        m, f = arrangement.mixer, arrangement.feed_forward
        w = self.keep[0]
        return (w[0] is m.w_qkv and w[1] is m.w_o and w[2] is f.w_gate_up and w[3] is f.w_down
                and self.keep[1][0] is arrangement.mixer_norm.weight and self.keep[1][1] is arrangement.feed_forward_norm.weight
                and bool(self.layer.mixer_partial) == bool(m.partial_output) and bool(self.layer.ff_partial) == bool(f.partial_output))

    def run(self, residual: torch.Tensor, delta: Optional[torch.Tensor], step, cache) -> Optional[torch.Tensor]:
        """The block's output (what the next norm adds to the residual), or None when the parts'
        own path has to run.  Nothing has been launched in that case."""
        if cache is None or cache.kind != "paged" or not cache.writes or cache.k.dtype != torch.bfloat16:
            return None
        sn = step.native
        if sn is None:
            sn = step.native = StepNative(step)
        if not sn.ok:
            return None
        T, H = sn.step.T, self.layer.H
        if residual.dtype != torch.float32 or residual.shape != (T, H) or not residual.is_contiguous():
            return None
        if delta is None:
            d_ptr, d_kind, d_splits = None, 0, 0
        elif delta.dim() == 2 and delta.dtype == torch.bfloat16 and delta.shape == (T, H) and delta.is_contiguous():
            d_ptr, d_kind, d_splits = delta.data_ptr(), 1, 0
        elif delta.dim() == 3 and delta.dtype == torch.float32 and delta.shape[1:] == (T, H) and delta.is_contiguous():
            d_ptr, d_kind, d_splits = delta.data_ptr(), 2, delta.shape[0]
        else:
            return None
        grp = sn.group(step, cache.group)
        if not grp:
            return None
        k, v = cache.k, cache.v
        if not (k.is_contiguous() and v.is_contiguous() and v.dtype == torch.bfloat16
                and tuple(k.shape[1:]) == (self.layer.nkv, cache.page_size, self.layer.hd) and v.shape == k.shape):
            return None
        call = _entry_point()
        head = (self.layer_ref, sn.step_ref, sn.tuning_ref, k.data_ptr(), v.data_ptr(), k.shape[0], cache.page_size,
                grp[0], grp[1], grp[2], residual.data_ptr(), d_ptr, d_kind, d_splits)
        plan = sn.plans.get(self.key)
        if plan is None:
            rc = call(*head, None, 0, 0, None, 0, 1, self.plan_ref)
            if rc == UNSUPPORTED:
                plan = False
            elif rc:
                self._raise(rc)
            else:
                s_ptr, s_bytes, _ = _scratch_for(sn.device, self.plan.scratch_bytes)
                plan = (self.plan.out_kind, self.plan.out_splits, s_ptr, s_bytes)
            sn.plans[self.key] = plan
        if plan is False:
            return None
        kind, splits, s_ptr, s_bytes = plan
        if kind == 2:
            out = torch.empty((splits, T, H), dtype=torch.float32, device=sn.device)
        else:
            out = torch.empty((T, H), dtype=torch.bfloat16, device=sn.device)
        rc = call(*head, out.data_ptr(), kind, splits, s_ptr, s_bytes, 0, self.plan_ref)
        if rc:
            self._raise(rc)
        global runs
        runs += 1
        return out

    def _raise(self, rc: int):
        lib = self.keep[3] if rc == ATTENTION_FAILED else ops.core()
        raise ops.KernelError(lib.coheryn_last_error().decode("utf-8", "replace"))
