"""Python face of the CUDA kernels: every function takes torch tensors that live on the
GPU, checks them, and launches a kernel of this package's own library on the current
CUDA stream.  There is no other implementation behind these functions: without a GPU
or without the compiled library they raise.
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_long, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float


class KernelError(RuntimeError):
    pass


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise KernelError("this engine runs on a CUDA GPU (sm_100a) only; "
                          "torch.cuda.is_available() is False and there is no CPU path")


_core = None
_attn_libs = {}


def core():
    global _core
    if _core is None:
        lib = build.core_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        lib.coheryn_argmax_scratch_slots.restype = ctypes.c_long
        lib.coheryn_gemm_tc_workspace_floats.restype = ctypes.c_long
        _core = lib
    return _core


def launch_count() -> int:
    """Kernel launches made through the core library since it was loaded."""
    return int(core().coheryn_launch_count())


def total_launch_count() -> int:
    """Kernel launches made through every library of this package that is loaded."""
    n = launch_count()
    for lib in _attn_libs.values():
        n += int(lib.coheryn_launch_count())
    return n


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not handled by the kernels") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


try:
    _raw_stream, _current_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:          # another torch: the documented, slower way
    _raw_stream = _current_device = None


def _stream():
    """The current CUDA stream of the current device as a pointer (asked on every launch: a few
    microseconds through ``torch.cuda.current_stream``, a tenth of one through the raw call)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(lib, rc: int) -> None:
    if rc != 0:
        raise KernelError(lib.coheryn_last_error().decode("utf-8", "replace"))


def _dev(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must be CUDA tensors")


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                 scale: Optional[float] = None) -> None:
    """out[t] = table[ids[t]] (* scale) as float32.  An id outside the table sets status to 1."""
    _dev(table, ids, out, status)
    _i32(ids, "ids")
    V, H = table.shape
    T = ids.numel()
    assert out.dtype == torch.float32 and out.shape == (T, H) and out.is_contiguous()
    assert table.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), c_int(T),
                                         c_int(H), c_int(V), _ptr(status), c_float(1.0 if scale is None else scale),
                                         _stream()))


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """src[rows] for a matrix (or a vector) whose rows are contiguous; ``rows`` int32 on the device."""
    _dev(src, rows)
    _i32(rows, "rows")
    R = rows.numel()
    if src.dim() == 1:
        out = torch.empty((R,), dtype=src.dtype, device=src.device)
        row_bytes, stride = src.element_size(), src.stride(0) * src.element_size()
    else:
        assert src.dim() == 2 and src.stride(1) == 1
        out = torch.empty((R, src.shape[1]), dtype=src.dtype, device=src.device)
        row_bytes, stride = src.shape[1] * src.element_size(), src.stride(0) * src.element_size()
    if R:
        lib = core()
        _check(lib, lib.coheryn_gather_rows(_ptr(src), c_long(stride), _ptr(rows), _ptr(out), c_int(R), c_int(row_bytes),
                                            _stream()))
    return out


def scatter_words(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[rows[r]] = src[r] for vectors of 32-bit elements."""
    _dev(src, rows, out)
    _i32(rows, "rows")
    assert src.element_size() == 4 and out.element_size() == 4 and src.is_contiguous() and out.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_scatter_words(_ptr(src), _ptr(rows), _ptr(out), c_int(rows.numel()), _stream()))


def scale_add_bias(x: torch.Tensor, scale: Optional[float], bias: Optional[torch.Tensor]) -> None:
    """In place on float32 rows: x = x * scale + bias (either may be absent)."""
    _dev(x, bias)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    if bias is not None:
        assert bias.shape == (x.shape[1],) and bias.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_scale_add_bias(_ptr(x), c_long(x.stride(0)), c_int(x.shape[0]), c_int(x.shape[1]),
                                           c_float(1.0 if scale is None else scale), _ptr(bias),
                                           c_int(_code(bias) if bias is not None else F32), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, update: bool = True) -> None:
    """x = resid (+ delta); resid = x if update; out = x / sqrt(mean(x^2) + eps) * weight.
    With ``rows`` only those rows are read (out[r] comes from row rows[r]) and the
    residual is left as it is.  ``delta`` may be a float32 stack [splits, n, H] of partial sums
    (see ``linear(partial_ok=True)``): they are added in order, then to the residual."""
    _dev(resid, delta, weight, out, rows)
    H = resid.shape[-1]
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert out.is_contiguous() and out.shape[-1] == H and weight.shape == (H,)
    n = out.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        assert rows.numel() == n
        update = False
    else:
        assert resid.shape[0] >= n
    lib = core()
    if delta is not None and delta.dim() == 3:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == resid.shape
        _check(lib, lib.coheryn_add_parts_rmsnorm(
            _ptr(resid), _ptr(delta), c_int(delta.shape[0]), c_long(delta.stride(0)), _ptr(rows), _ptr(weight),
            c_int(_code(weight)), c_float(eps), _ptr(out), c_int(_code(out)), c_int(n), c_int(H),
            c_int(1 if update else 0), _stream()))
        return
    if delta is not None:
        assert delta.is_contiguous() and delta.shape == resid.shape
    _check(lib, lib.coheryn_add_rmsnorm(
        _ptr(resid), _ptr(delta), c_int(_code(delta) if delta is not None else F32), _ptr(rows),
        _ptr(weight), c_int(_code(weight)), c_float(eps), _ptr(out), c_int(_code(out)), c_int(n),
        c_int(H), c_int(1 if (update and delta is not None) else 0), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[m, j] = silu(gate_up[m, 2j]) * gate_up[m, 2j + 1] (gate and up interleaved)."""
    _dev(gate_up, out)
    M, I2 = gate_up.shape
    assert I2 % 2 == 0 and out.shape == (M, I2 // 2) and out.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and out.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_silu_mul(_ptr(gate_up), _ptr(out), c_int(_code(out)), c_int(M),
                                     c_int(I2 // 2), _stream()))


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                  slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  rotary_dim: int, page_size: int) -> None:
    """Rotate q (in place) and k by position; write rotated k and v into cache pages
    laid out [page, kv head, slot, head_dim] at ``slots`` (page * page_size + offset).
    Without caches (a layer that reads another layer's cache) the buffer holds query
    heads only and they are rotated in place."""
    _dev(qkv, positions, cos_sin, slots, k_cache, v_cache)
    _i32(positions, "positions")
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    if rotary_dim:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
        assert cos_sin.shape[1:] == (rotary_dim // 2, 2)
    write = k_cache is not None
    if write:
        _i32(slots, "slots")
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
    else:
        assert num_kv_heads == 0, "without a cache to write, only query heads are rotated"
    lib = core()
    _check(lib, lib.coheryn_rope_kv_write(
        _ptr(qkv), c_int(_code(qkv)), _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(k_cache),
        _ptr(v_cache), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(rotary_dim), c_int(page_size), c_int(1 if write else 0), _stream()))


# Up to this many rows the q/k/v product rotates and writes the cache in its own epilogue.
QKV_ROPE_M = int(os.environ.get("COHERYN_QKV_ROPE_M", "16"))


def qkv_rope_ok(x, w_qkv, k_cache, rotary_dim: int, head_dim: int) -> bool:
    return (0 < x.shape[0] <= QKV_ROPE_M and x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
            and k_cache is not None and k_cache.dtype == torch.bfloat16 and rotary_dim == head_dim
            and head_dim % 16 == 0 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w_qkv.is_contiguous() and w_qkv.data_ptr() % 16 == 0)


def qkv_rope_small(x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], positions: torch.Tensor,
                   cos_sin: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> torch.Tensor:
    """q, k, v = x @ w_qkv.T (+ b) for at most 16 rows with the rotation of q and k and the
    cache write of k and v in the product's epilogue (see ``rope_kv_write`` for the layout).
    Returns the rotated q ``[T, num_heads * head_dim]``; the whole head is rotated."""
    _dev(x, w_qkv, b_qkv, positions, cos_sin, slots, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slots, "slots")
    T, K = x.shape
    assert w_qkv.shape == ((num_heads + 2 * num_kv_heads) * head_dim, K)
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (head_dim // 2, 2)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
    q = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    lib = core()
    _check(lib, lib.coheryn_qkv_rope_bf16_small(
        _ptr(x), _ptr(w_qkv), _ptr(b_qkv), c_int(_code(b_qkv) if b_qkv is not None else F32), _ptr(q),
        c_long(q.stride(0)), _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(T),
        c_int(K), c_long(x.stride(0)), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        _stream()))
    return q


def seeded_fill(out: torch.Tensor, key: int, first: int, mean: float, deviation: float) -> None:
    """out.flatten()[i] = the seeded random value of element first + i of the tensor with ``key``
    (see weights/seeded.py), float32 or bfloat16."""
    _dev(out)
    assert out.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_seeded_fill(_ptr(out), c_int(_code(out)), ctypes.c_ulonglong(key), ctypes.c_ulonglong(first),
                                        ctypes.c_ulonglong(out.numel()), ctypes.c_double(mean), ctypes.c_double(deviation),
                                        _stream()))


# Up to this many rows a q/k/v product whose K the many-rows kernel splits leaves the addition of
# its slices to the rotation kernel (one kernel less between the product and the attention).
QKV_PARTS_M = int(os.environ.get("COHERYN_QKV_PARTS_M", "256"))
# ... by the few-rows product above this many rows (up to FEW_DEFER_M), by the many-rows product otherwise
# (at 64 rows the latter is 2 % of a decode step faster).
QKV_PARTS_FEW_FROM = 64


def qkv_parts_count(x, w_qkv, k_cache, rotary_dim: int, head_dim: int) -> int:
    """The K slices that ``qkv_rope_parts`` would leave for this step's q/k/v product (0: not that path)."""
    M, K = x.shape
    if not (QKV_ROPE_M < M <= QKV_PARTS_M and x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
            and k_cache is not None and k_cache.dtype == torch.bfloat16 and rotary_dim == head_dim and head_dim % 16 == 0
            and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w_qkv.is_contiguous()
            and w_qkv.data_ptr() % 16 == 0):
        return 0
    few = few_splits(w_qkv.shape[0], K)           # the few-rows product (weights streamed once) where it cuts K
    if few > 1 and QKV_PARTS_FEW_FROM < M <= FEW_DEFER_M:
        return few
    return int(core().coheryn_gemm_tc_parts_count(c_int(M), c_int(w_qkv.shape[0]), c_int(K)))


def qkv_rope_parts(x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], positions: torch.Tensor,
                   cos_sin: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, count: int) -> torch.Tensor:
    """q, k, v = x @ w_qkv.T (+ b) by the few-rows product (or, where that does not cut K, the many-rows
    product) with K cut into ``count`` slices, whose
    addition, the bias, the rotation of q and k and the cache write of k and v happen in ONE following
    kernel (see ``rope_kv_write``).  Returns the rotated q ``[T, num_heads * head_dim]``."""
    _dev(x, w_qkv, b_qkv, positions, cos_sin, slots, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slots, "slots")
    T, K = x.shape
    N = w_qkv.shape[0]
    assert N == (num_heads + 2 * num_kv_heads) * head_dim
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (head_dim // 2, 2)
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
    lib = core()
    parts = torch.empty((count, T, N), dtype=torch.float32, device=x.device)
    if count == few_splits(N, K):
        gemm_bf16_tc_few(x, w_qkv, None, parts, defer=True)
    else:
        _check(lib, lib.coheryn_gemm_bf16_tc_parts(_ptr(x), _ptr(w_qkv), _ptr(parts), c_int(T), c_int(N), c_int(K),
                                                   c_long(x.stride(0)), _ptr(tc_status(x.device)), _stream()))
    q = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    _check(lib, lib.coheryn_rope_kv_write_parts(
        _ptr(parts), c_int(count), c_long(T * N), _ptr(b_qkv), c_int(_code(b_qkv) if b_qkv is not None else F32), _ptr(q),
        _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_int(page_size), _stream()))
    return q


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ w.T (+ bias) with float32 FMA accumulation (no tensor cores)."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and w.is_contiguous() and out.shape == (M, N)
    assert x.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert bias.shape == (N,) and bias.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_gemm_simt(
        _ptr(x), c_int(_code(x)), _ptr(w), c_int(_code(w)), _ptr(bias),
        c_int(_code(bias) if bias is not None else F32), _ptr(out), c_int(_code(out)), c_int(M),
        c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)), _stream()))


def attention_simple(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                     num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                     window: Optional[int], scale: float) -> None:
    """Causal attention of each token over its request's cache pages (float32 math).
    ``q`` may be a column slice of a wider buffer (its row stride is honoured)."""
    _dev(q, out, k_cache, v_cache, block_tables, token_req, positions)
    _i32(block_tables, "block_tables"); _i32(token_req, "token_req"); _i32(positions, "positions")
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim
    assert k_cache.dtype == q.dtype and out.dtype == q.dtype
    lib = core()
    _check(lib, lib.coheryn_attention_simple(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(_code(q)), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(token_req),
        _ptr(positions), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window or 0), c_float(scale), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[r] = lowest index of the maximum of logits[r]; non-finite logits set status 2."""
    _dev(logits, out, status)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _i32(out, "out")
    lib = core()
    slots = int(lib.coheryn_argmax_scratch_slots(c_int(R), c_int(V)))
    scratch = torch.empty(2 * slots, dtype=torch.int32, device=logits.device) if slots else None
    _check(lib, lib.coheryn_argmax(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V),
                                   _ptr(out), _ptr(status), _ptr(scratch), c_long(slots), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """Temperature / top-k / top-p sampling of one token per row from host-made draws."""
    _dev(logits, temperature, top_k, top_p, uniform, out, status)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert uniform.dtype == torch.float64
    _i32(top_k, "top_k"); _i32(out, "out")
    lib = core()
    _check(lib, lib.coheryn_sample(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V),
                                   _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
                                   _ptr(out), _ptr(status), _stream()))


def apply_penalties(logits, rows, ids, counts, rep, freq, pres) -> None:
    """In place: the reference's penalties on logits[rows[i], ids[i]] (each pair once)."""
    _dev(logits, rows, ids, counts, rep, freq, pres)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    for t in (rows, ids, counts):
        _i32(t, "penalty index")
    lib = core()
    _check(lib, lib.coheryn_apply_penalties(_ptr(logits), c_long(logits.stride(0)), c_int(rows.numel()),
                                            _ptr(rows), _ptr(ids), _ptr(counts), _ptr(rep), _ptr(freq),
                                            _ptr(pres), _stream()))


# ------------------------------------------------------------------------------------
def gemm_bf16_small(x, w, bias, out, gated: int = 0) -> None:
    """Tensor-core product for at most 64 rows (decode); see csrc/gemm_bf16_small.cu."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    lib = core()
    _check(lib, lib.coheryn_gemm_bf16_small(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)),
        c_int(int(gated)), _stream()))


# Up to this many rows the weight-streaming mma.sync kernel runs; beyond it the TMA/tcgen05
# kernel (which re-reads nothing of x through L2 and so scales to many rows).
SMALL_M = 16
_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """Device word that the tensor-core GEMM sets when one of its bounded waits runs out."""
    t = _tc_status.get(device)
    if t is None:
        t = _tc_status[device] = _tc_status.setdefault(str(torch.device(device)), torch.zeros(1, dtype=torch.int32, device=device))
    return t


STATUS_MESSAGES = {1: "a token id was outside the embedding table", 2: "non-finite logits"}


def describe_status(code: int) -> str:
    """What a non-zero device status word means."""
    if code in STATUS_MESSAGES:
        return STATUS_MESSAGES[code]
    if 11 <= code <= 39:
        return (f"a kernel gave up a bounded wait and left its output unfinished (code {code}: 11-13 tensor-core product: "
                "producer, MMA issuer, epilogue; 19 self-test; 31-39 prompt attention: 31 producer, 32-36 MMA issuer, "
                "37-39 softmax)")
    return f"device status {code}"


def check_tc_status(device) -> None:
    code = int(tc_status(device).item())
    if code:
        tc_status(device).zero_()
        raise KernelError(describe_status(code))


def selftest_bounded_wait(device, tries: int = 300, code: int = 19) -> None:
    """Launch the self-test kernel: it waits ``tries`` times on a barrier nothing arrives on, gives
    up, and records ``code`` in the status word of the tensor-core kernels (see csrc/selftest.cu)."""
    lib = core()
    _check(lib, lib.coheryn_selftest_bounded_wait(_ptr(tc_status(device)), ctypes.c_uint(tries), c_int(code), _stream()))


def gemm_bf16_tc(x, w, bias, out, gated: int = 0) -> None:
    """TMA + tcgen05 product for many rows (prompt portions); see csrc/gemm_tc.cu."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    lib = core()
    floats = _tc_workspace_floats(M, N, K)   # > 0: K is split
    workspace = torch.empty(floats, dtype=torch.float32, device=x.device) if floats else None
    _check(lib, lib.coheryn_gemm_bf16_tc(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)),
        c_int(int(gated)), _ptr(tc_status(x.device)), _ptr(workspace), c_long(floats), _stream()))


def set_gemm_pairs(on: bool) -> None:
    """Whether ``gemm_bf16_tc`` hands suitable shapes to the kernel of CTA pairs (default: yes)."""
    core().coheryn_gemm_tc_set_pairs(c_int(1 if on else 0))
    _tc_workspace_floats.cache_clear()      # the pairs take shapes that would otherwise split K


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """K splits that ``gemm_bf16_tc`` uses for this shape (1: none; a shape run by CTA pairs: 1)."""
    return max(1, _tc_workspace_floats(M, N, K) // (M * N))


def gemm_bf16_tc_pair(x, w, bias, out, gated: int = 0) -> None:
    """The many-rows product by pairs of CTAs sharing 256 x 256 tiles (tcgen05 cta_group::2);
    see gemm_tc_pair_kernel in csrc/gemm_tc.cu."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    lib = core()
    _check(lib, lib.coheryn_gemm_bf16_tc_pair(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)),
        c_int(int(gated)), _ptr(tc_status(x.device)), _stream()))


_few_workspaces = {}
_few_retired = []     # outgrown workspaces stay alive: captured graphs may still name them


def _few_workspace(device, floats: int) -> torch.Tensor:
    """Zero-initialised scratch of the few-rows product: counters, then the K splits' tiles.
    One per device: the products that share it must run in stream order on one stream."""
    key = str(device)
    ws = _few_workspaces.get(key)
    if ws is None or ws.numel() < floats:
        if ws is not None:
            _few_retired.append(ws)
        ws = torch.zeros(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _few_workspaces[key] = ws
    return ws


@functools.lru_cache(maxsize=None)
def few_splits(N: int, K: int) -> int:
    """Into how many slices of K the few-rows product cuts this weight shape (1: none)."""
    return int(core().coheryn_gemm_tc_few_splits(c_int(N), c_int(K)))


@functools.lru_cache(maxsize=None)
def _tc_workspace_floats(M: int, N: int, K: int) -> int:
    return int(core().coheryn_gemm_tc_workspace_floats(c_int(M), c_int(N), c_int(K)))


@functools.lru_cache(maxsize=None)
def _few_workspace_floats(M: int, N: int, K: int) -> int:
    return int(core().coheryn_gemm_tc_few_workspace_floats(c_int(M), c_int(N), c_int(K)))


def gemm_bf16_tc_few(x, w, bias, out, gated: int = 0, defer: bool = False) -> None:
    """TMA + tcgen05 product for at most 64 rows with the features on the accumulator's
    lanes (decode, short portions); see csrc/gemm_tc_few.cu.  ``defer``: ``out`` is a float32
    stack [splits, M, N] of the K slices' sums, left for the consumer to add."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(-1) == 1
    lib = core()
    if defer:
        assert not gated and out.dtype == torch.float32 and out.is_contiguous()
        assert out.shape == (few_splits(N, K), M, N)
        floats = 0
    else:
        assert out.shape == (M, N // 2 if gated else N)
        floats = _few_workspace_floats(M, N, K)   # > 0: K is split
    workspace = _few_workspace(x.device, floats) if floats else None
    _check(lib, lib.coheryn_gemm_bf16_tc_few(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(-2)),
        c_int(int(gated)), _ptr(tc_status(x.device)), _ptr(workspace),
        c_long(workspace.numel() if workspace is not None else 0), c_int(1 if defer else 0), _stream()))


# Up to this many rows the few-rows tcgen05 kernel takes the products whose K it need not
# split, or whose consumer adds the splits (0 switches it off).  A product that would have to
# add its own splits goes to the mma.sync kernel instead: measured on a B200, the in-kernel
# addition through memory costs several dependent round trips.
FEW_M = int(os.environ.get("COHERYN_FEW_M", "32"))
# ... and up to this many rows the products whose K slices the consumer adds.  The kernel takes up to
# 256 rows, but every CTA re-reads all rows of x beside its weight tile, and from 129 rows on that costs
# what the many-rows kernel with its extra kernel for the K slices costs (1.5B sizes, down projection:
# 128 rows 15.9 -> 12.7 us, 256 rows 21.1 -> 18.8; a decode step at batch 128 3.64 -> 3.45 ms, at 256 no change).
FEW_DEFER_M = int(os.environ.get("COHERYN_FEW_DEFER_M", "128"))
# The output head (a very large weight) takes the few-rows product up to this many rows only: every CTA
# re-reads all rows of x, which beyond that costs more than the weight stream.
FEW_HEAD_M = 64


# A product hands its K slices to the consumer only from this K on.  Measured on a B200 at 8
# rows: for K = 1536 (12 slices of two steps) the norm that adds twelve parts loses more than
# the product gains over the mma.sync kernel; for K = 8960 the pair is 5 us faster.
DEFER_MIN_K = 4096
# With more than SMALL_M_SHORT rows the alternative is the many-rows kernel plus the kernel that adds
# its K splits: there the slices pay from K = 1024 on (1 % of a decode step at 40 and 64 rows).
DEFER_MIN_K_WIDE = int(os.environ.get("COHERYN_DEFER_MIN_K_WIDE", "1024"))


# A weight matrix of at least this many elements (the output head over a large vocabulary) goes
# through the few-rows product up to FEW_HEAD_M rows: its stream is all that matters there.
FEW_LARGE_WEIGHT = 128 << 20


def _few_ok(x, w, partial_ok: bool = False) -> bool:
    if not _few_shape_ok(x, w, FEW_HEAD_M if w.numel() >= FEW_LARGE_WEIGHT else None):
        return False
    return partial_ok or few_splits(w.shape[0], w.shape[1]) == 1


def _few_shape_ok(x, w, limit: Optional[int] = None) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= (FEW_M if limit is None else limit)
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def _tc_ok(x, w) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > SMALL_M
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


# ... and up to this many rows when the weight matrix is small (a few MB: the q/k/v and output
# products of a decode batch), where one launch of the mma.sync kernel beats the tcgen05 kernel
# plus the kernel that adds its K splits.
SMALL_M_SHORT = int(os.environ.get("COHERYN_SMALL_M_SHORT", "32"))
SMALL_WEIGHT_ELEMENTS = 4 << 20


def _small_ok(x, w) -> bool:
    M = x.shape[0]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and (0 < M <= SMALL_M or (0 < M <= SMALL_M_SHORT and w.numel() <= SMALL_WEIGHT_ELEMENTS))
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
           partial_ok: bool = False) -> torch.Tensor:
    """y = x @ w.T (+ bias), float32 accumulation.  float32 operands use FMA on the CUDA
    cores (no reduced-precision tensor mode); bfloat16 operands use the tensor-core
    kernels where the shape allows and the FMA kernel otherwise.  With ``partial_ok`` the
    result may come as a float32 stack [splits, M, N] of partial sums whose addition is left
    to the consumer (``add_rmsnorm`` takes such a stack as its delta)."""
    M, N = x.shape[0], w.shape[0]
    if (partial_ok and out is None and M and w.shape[1] >= (DEFER_MIN_K_WIDE if M > SMALL_M_SHORT else DEFER_MIN_K)
            and _few_shape_ok(x, w, FEW_DEFER_M)):
        splits = few_splits(N, w.shape[1])
        if splits > 1:
            parts = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
            gemm_bf16_tc_few(x, w, bias, parts, defer=True)
            return parts
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    if _few_ok(x, w):
        gemm_bf16_tc_few(x, w, bias, out)
    elif _small_ok(x, w):
        gemm_bf16_small(x, w, bias, out)
    elif _tc_ok(x, w):
        gemm_bf16_tc(x, w, bias, out)
    else:
        gemm_simt(x, w, bias, out)
    return out


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step,
              group: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
              window: Optional[int], scale: float) -> None:
    """Attention of every token of the step over its request's cache pages of ``group``
    (``step`` is a StepContext).  Chooses the kernel by dtype and shape."""
    attention_rows(q, out, k_cache, v_cache, step.block_tables[group], step.token_req,
                   step.positions, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                   cu_q=step.cu_q, kv_lens=step.kv_lens, q_lens=step.q_lens, max_kv_len=step.max_kv_len,
                   settled=step.prior_positions_settled)


def attention_lib(head_dim: int):
    lib = _attn_libs.get(head_dim)
    if lib is None:
        lib = build.attention_library(head_dim)
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_attn_scratch_floats.restype = ctypes.c_long
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        if lib.coheryn_attn_head_dim() != head_dim:
            raise KernelError(f"attention library was built for head size {lib.coheryn_attn_head_dim()}, not {head_dim}")
        _attn_libs[head_dim] = lib
    return lib


def set_attention_split(head_dim: int, keys: int) -> None:
    """Fix the positions per CTA of the decode attention kernel for this head size (a power of two
    from 128 to 2048, capped at 256 pages); 0 restores the choice by batch size and context.  For tests and experiments."""
    attention_lib(head_dim).coheryn_attn_set_split(c_int(keys))


def set_attention_tc_two_tiles(head_dim: int, on: Optional[bool]) -> None:
    """Whether the prompt-portion attention kernel gives a CTA two consecutive row tiles that share
    every fetched key tile (head sizes up to 128): always, never, or (None, the default) when the
    pairs still fill the GPU.  For tests and experiments."""
    attention_lib(head_dim).coheryn_attn_set_tc_two_tiles(c_int(2 if on is None else (1 if on else 0)))


def set_attention_tc_cluster(head_dim: int, cluster: int) -> None:
    """Fix the number of CTAs (1, 2, 4 or 8) that share a row tile of the prompt-portion attention
    kernel and split its keys; 0 restores the choice by shape.  For tests and experiments."""
    attention_lib(head_dim).coheryn_attn_set_tc_cluster(c_int(cluster))


def attention_rows(q, out, k_cache, v_cache, block_tables, token_req, positions, num_heads, num_kv_heads,
                   head_dim, page_size, window, scale, cu_q=None, kv_lens=None, q_lens=None,
                   max_kv_len=None, force_simple=False, settled=True) -> None:
    """Attention of rows (request token_req[i] at position positions[i]) over cache pages.
    bfloat16 rows that are whole runs of consecutive positions per request, ending at the
    request's last position (``cu_q``, ``kv_lens`` on the device, ``q_lens`` and
    ``max_kv_len`` on the host) go to the tensor-core kernels when the head size is a
    multiple of 16 up to 256; everything else goes to the float32-arithmetic kernel.
    ``settled``: the keys and values at positions before each request's first row were written by
    earlier steps, so the decode kernel may fetch them before it waits for the step's earlier
    kernels; False when this step itself wrote them (the wanted rows of a portion)."""
    fast = (not force_simple and q.dtype == torch.bfloat16 and cu_q is not None and kv_lens is not None
            and q_lens is not None and max_kv_len is not None and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and q.stride(0) % 8 == 0 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0)
    if not fast:
        attention_simple(q, out, k_cache, v_cache, block_tables, token_req, positions, num_heads,
                         num_kv_heads, head_dim, page_size, window, scale)
        return
    _dev(q, out, k_cache, v_cache, block_tables, cu_q, kv_lens)
    _i32(block_tables, "block_tables"); _i32(cu_q, "cu_q"); _i32(kv_lens, "kv_lens")
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == q.dtype and k_cache.dtype == q.dtype
    G = num_heads // num_kv_heads
    B = len(q_lens)
    rows = [n * G for n in q_lens]
    any_small = any(r <= 16 for r in rows)
    any_large = any(r > 16 for r in rows)
    lib = attention_lib(head_dim)
    scratch, floats = None, 0
    if any_small and G <= 16:
        floats = int(lib.coheryn_attn_scratch_floats(c_int(B), c_int(num_kv_heads), c_int(max_kv_len)))
        scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    _check(lib, lib.coheryn_attention_bf16(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_q), _ptr(kv_lens), c_int(B),
        c_int(num_heads), c_int(num_kv_heads), c_int(page_size), c_int(window or 0), c_float(scale),
        c_int(max(rows)), c_int(1 if any_small else 0), c_int(1 if any_large else 0), c_int(max_kv_len),
        _ptr(scratch), c_long(floats), _ptr(tc_status(q.device)), c_int(q.shape[0]), c_int(k_cache.shape[0]),
        c_int(1 if settled else 0), _stream()))


# Decode steps of at most this many requests merge the attention splits inside the output
# projection's kernel (0 switches that off: the splits are merged by a kernel of their own and the
# projection is an ordinary product).
ATTN_OPROJ_M = int(os.environ.get("COHERYN_ATTN_OPROJ_M", "16"))


# ... and only while the merging stays cheap: every CTA of the merged kernel (one per head and tile of
# 128 output features) reads the splits of its head for all requests again, so the bytes read grow with
# width / 128 x heads x requests x splits.  Beyond this many bytes the splits are merged once, by the
# kernel of their own.
ATTN_OPROJ_MERGE_BYTES = int(os.environ.get("COHERYN_ATTN_OPROJ_BYTES", str(32 << 20)))


# Whether a pre-norm block made of the built-in parts is enqueued by one call into the library
# (csrc/block_runner.cu) instead of part by part; the kernels and their order are the same.
NATIVE_BLOCK = os.environ.get("COHERYN_NATIVE_BLOCK", "1") != "0"


def set_native_block(on: bool) -> None:
    global NATIVE_BLOCK
    NATIVE_BLOCK = bool(on)


def attention_oproj_ok(q: torch.Tensor, w_o: torch.Tensor, step, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    if step.max_kv_len is None or step.max_q_len != 1:
        return False
    tiles = -(-w_o.shape[0] // 128)
    merge_bytes = tiles * num_heads * step.num_requests * (-(-step.max_kv_len // 128)) * head_dim * 4
    return (merge_bytes <= ATTN_OPROJ_MERGE_BYTES and q.dtype == torch.bfloat16 and w_o.dtype == torch.bfloat16 and step.max_q_len == 1
            and 0 < step.num_requests <= min(ATTN_OPROJ_M, 16) and q.shape[0] == step.num_requests
            and num_heads // num_kv_heads <= 16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and step.max_kv_len is not None and (step.max_kv_len + 127) // 128 + 1 <= 512
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and w_o.stride(1) == 1 and w_o.stride(0) % 8 == 0
            and w_o.data_ptr() % 16 == 0 and w_o.shape[0] % 4 == 0)


def attention_oproj(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step, group: int, num_heads: int,
                    num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int], scale: float,
                    w_o: torch.Tensor, b_o: Optional[torch.Tensor]) -> torch.Tensor:
    """Decode attention of one token per request and the output projection: returns a float32 stack
    [num_heads, B, H] whose sum over the heads is attention(q) @ w_o.T (+ b_o); the consumer (a norm
    that takes partial sums) adds the heads in order.  See attn_merge_oproj in csrc/attention_bf16.cu."""
    block_tables, cu_q, kv_lens = step.block_tables[group], step.cu_q, step.kv_lens
    _dev(q, k_cache, v_cache, block_tables, cu_q, kv_lens, w_o, b_o)
    _i32(block_tables, "block_tables"); _i32(cu_q, "cu_q"); _i32(kv_lens, "kv_lens")
    B, H = step.num_requests, w_o.shape[0]
    assert w_o.shape[1] == num_heads * head_dim and k_cache.dtype == q.dtype
    lib = attention_lib(head_dim)
    floats = int(lib.coheryn_attn_scratch_floats(c_int(B), c_int(num_kv_heads), c_int(step.max_kv_len)))
    scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    parts = torch.empty((num_heads, B, H), dtype=torch.float32, device=q.device)
    _check(lib, lib.coheryn_attention_oproj_bf16(
        _ptr(q), c_long(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(cu_q), _ptr(kv_lens), c_int(B), c_int(num_heads), c_int(num_kv_heads), c_int(page_size), c_int(window or 0),
        c_float(scale), c_int(step.max_kv_len), _ptr(scratch), c_long(floats), _ptr(w_o), c_long(w_o.stride(0)), c_int(H),
        _ptr(b_o), c_int(_code(b_o) if b_o is not None else F32), _ptr(parts), c_int(1 if step.prior_positions_settled else 0),
        _stream()))
    return parts


# Activations of the gated epilogue, by the code that the kernels take as their ``gated`` argument
# (0 means "no gate").  The gate is applied in float32 inside the product's epilogue; an activation
# that is not built is refused here by name, before anything is launched.
GATED_ACTIVATIONS = {"silu": 1}


def gated_activation_code(activation: str) -> int:
    try:
        return GATED_ACTIVATIONS[activation]
    except KeyError:
        raise KernelError(f"the gated epilogue of the matrix products is not built for activation {activation!r} "
                          f"(built: {', '.join(sorted(GATED_ACTIVATIONS))})") from None


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """act(x @ Wg.T) * (x @ Wu.T) for w_gate_up with INTERLEAVED rows (row 2j = gate_j,
    row 2j+1 = up_j), so that a gate/up pair lands in one thread of the epilogue."""
    code = gated_activation_code(activation)
    M = x.shape[0]
    I = w_gate_up.shape[0] // 2
    out = torch.empty((M, I), dtype=x.dtype, device=x.device)
    if M == 0:
        return out
    if _few_ok(x, w_gate_up):
        gemm_bf16_tc_few(x, w_gate_up, None, out, gated=code)
        return out
    if _small_ok(x, w_gate_up):
        gemm_bf16_small(x, w_gate_up, None, out, gated=code)
        return out
    if _tc_ok(x, w_gate_up):
        gemm_bf16_tc(x, w_gate_up, None, out, gated=code)
        return out
    gu = torch.empty((M, 2 * I), dtype=x.dtype, device=x.device)
    gemm_simt(x, w_gate_up, None, gu)
    silu_mul(gu, out)
    return out
