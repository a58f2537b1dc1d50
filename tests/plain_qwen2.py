"""A plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache, one
function for each part, numpy only.  It shares no code with the engine (it even reads
safetensors by itself) and is the yardstick of every engine test.

It rests on the reference's formulas, cited per function by file:line within
Coheryn/coheryn-ai-studio.  The reference's Rust code cannot be compiled or imported here
(no Rust toolchain), so it is anchored instead on the reference's weight-free fixtures
(fixtures/quantized/rope.json, fixtures/constraints/sampling-v2.json) and on the literal
values of its unit tests (crates/coheryn-engine/src/cpu.rs:229-256); see
tests/test_plain.py.

Precision: values are float32; every reduction (dot products, the norm's sum of squares,
the softmax denominator, the probability-weighted sum of values) is accumulated in
float64 and rounded to float32, as crates/coheryn-engine/src/cpu.rs:31-35, 51, 178-196
do.  (One deviation, far below any tolerance used: the reference rounds each product to
float32 before the float64 sum; here products of float32 values are exact in float64.)
"""
from __future__ import annotations

import json
import struct
from typing import Dict, Optional

import numpy as np

f32 = np.float32


# ------------------------------------------------------------------------------ files
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """name -> float32 (or int32) array.  BF16 is widened exactly."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        payload = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = payload[b:e]
        dt = info["dtype"]
        if dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(f32)
        elif dt == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(f32)
        elif dt == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(f32)
        elif dt == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = a.reshape(info["shape"])
    return out


def read_model(model_dir: str):
    with open(f"{model_dir}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{model_dir}/model.safetensors")


# ------------------------------------------------------------------------------ parts
def embedding(table: np.ndarray, ids) -> np.ndarray:
    """x = E[token] (crates/coheryn-engine/src/inference.rs:426-432)."""
    ids = np.asarray(ids)
    if ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token ID outside vocabulary")
    return table[ids].astype(f32)


def linear(x: np.ndarray, w: np.ndarray, b: Optional[np.ndarray] = None) -> np.ndarray:
    """y = W x (+ b): float64 sum rounded to float32, bias added after in float32
    (crates/coheryn-engine/src/cpu.rs:31-35; crates/coheryn-engine/src/inference.rs:450-471)."""
    y = (x.astype(np.float64) @ w.astype(np.float64).T).astype(f32)
    if b is not None:
        y = (y + b.astype(f32)).astype(f32)
    return y


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """mean = (sum x^2 in float64 / n) as f32; scale = 1/sqrt(mean + eps); y = (x*scale)*w
    (crates/coheryn-engine/src/cpu.rs:49-57)."""
    x = x.astype(f32)
    sq = (x * x).astype(f32).astype(np.float64)
    mean = (sq.sum(axis=-1, keepdims=True) / x.shape[-1]).astype(f32)
    scale = (f32(1.0) / np.sqrt(mean + f32(eps), dtype=f32)).astype(f32)
    return ((x * scale).astype(f32) * w.astype(f32)).astype(f32)


def rope_angles(position: int, head_dim: int, theta: float) -> np.ndarray:
    """angle_0 = position; angle_{i+1} = angle_i * theta**(-2/head_dim), all in float32
    (crates/coheryn-engine/src/cpu.rs:59-70)."""
    step = f32(np.power(f32(theta), f32(-2.0) / f32(head_dim)))
    out = np.empty(head_dim // 2, dtype=f32)
    angle = f32(position)
    for i in range(head_dim // 2):
        out[i] = angle
        angle = f32(angle * step)
    return out


def rope(x: np.ndarray, positions, head_dim: int, theta: float) -> np.ndarray:
    """Rotate-half per head: (a, b) = (h[i], h[i + d/2]);
    h[i] = a cos - b sin; h[i + d/2] = a sin + b cos (crates/coheryn-engine/src/cpu.rs:58-73).
    x: [T, heads * head_dim]."""
    T = x.shape[0]
    half = head_dim // 2
    h = x.astype(f32).reshape(T, -1, head_dim).copy()
    for t in range(T):
        ang = rope_angles(int(positions[t]), head_dim, theta)
        c, s = np.cos(ang, dtype=f32), np.sin(ang, dtype=f32)
        a, b = h[t, :, :half].copy(), h[t, :, half:].copy()
        # f32::mul_add rounds once: evaluate in float64 and round.
        h[t, :, :half] = (a.astype(np.float64) * c - (b * s).astype(f32).astype(np.float64)).astype(f32)
        h[t, :, half:] = (a.astype(np.float64) * s + (b * c).astype(f32).astype(np.float64)).astype(f32)
    return h.reshape(T, -1)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, heads: int, kv_heads: int, head_dim: int,
              window: Optional[int] = None) -> np.ndarray:
    """For head h of group h // (heads / kv_heads): s_t = (q . K_t) / sqrt(d) over t <= p,
    e_t = exp(s_t - max) in float32, den = sum e_t in float64, P_t = e_t * (1/den) as f32,
    o = sum_t P_t V_t in float64, rounded (crates/coheryn-engine/src/cpu.rs:133-210).  The
    mask is the explicit [T, T] lower triangle (the reference's cache holds only positions
    <= p); ``window`` additionally hides t <= p - window."""
    T = q.shape[0]
    qh = q.reshape(T, heads, head_dim)
    kh = k.reshape(T, kv_heads, head_dim)
    vh = v.reshape(T, kv_heads, head_dim)
    scale = f32(1.0) / np.sqrt(f32(head_dim), dtype=f32)
    out = np.zeros((T, heads, head_dim), dtype=f32)
    rows, cols = np.arange(T)[:, None], np.arange(T)[None, :]
    visible = cols <= rows
    if window is not None:
        visible &= cols > rows - window
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = ((qh[:, h].astype(np.float64) @ kh[:, g].astype(np.float64).T).astype(f32) * scale).astype(f32)
        s = np.where(visible, s, f32(-np.inf))
        m = s.max(axis=-1, keepdims=True)
        e = np.exp((s - m).astype(f32), dtype=f32)
        den = e.astype(np.float64).sum(axis=-1, keepdims=True)
        p = (e * (1.0 / den).astype(f32)).astype(f32)
        out[:, h] = (p.astype(np.float64) @ vh[:, g].astype(np.float64)).astype(f32)
    return out.reshape(T, heads * head_dim)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """a = (g / (1 + exp(-g))) * u in float32 (crates/coheryn-engine/src/cpu.rs:74-78)."""
    g = gate.astype(f32)
    return ((g / (f32(1.0) + np.exp(-g, dtype=f32))).astype(f32) * up.astype(f32)).astype(f32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16 (ties to even), kept as float32."""
    u = np.ascontiguousarray(x, dtype=f32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(f32)


def decoder_layer(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, cfg: dict, positions,
                  window: Optional[int] = None, rnd=None) -> np.ndarray:
    """Pre-norm residual block (crates/coheryn-engine/src/inference.rs:440-540).  ``rnd`` (None: the
    identity) is applied to what a part hands to the next: see ``forward``."""
    rnd = rnd or (lambda a: a)
    heads, kv_heads = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // heads
    eps, theta = cfg["rms_norm_eps"], cfg.get("rope_theta", 10000.0)
    g = lambda n: w.get(f"{prefix}.{n}")
    y = rnd(rms_norm(x, g("input_layernorm.weight"), eps))
    q = rnd(linear(y, g("self_attn.q_proj.weight"), g("self_attn.q_proj.bias")))
    k = rnd(linear(y, g("self_attn.k_proj.weight"), g("self_attn.k_proj.bias")))
    v = rnd(linear(y, g("self_attn.v_proj.weight"), g("self_attn.v_proj.bias")))
    q, k = rnd(rope(q, positions, hd, theta)), rnd(rope(k, positions, hd, theta))
    o = rnd(attention(q, k, v, heads, kv_heads, hd, window))
    x = (x + rnd(linear(o, g("self_attn.o_proj.weight")))).astype(f32)
    y = rnd(rms_norm(x, g("post_attention_layernorm.weight"), eps))
    a = rnd(swiglu(linear(y, g("mlp.gate_proj.weight")), linear(y, g("mlp.up_proj.weight"))))
    return (x + rnd(linear(a, g("mlp.down_proj.weight")))).astype(f32)


def forward(cfg: dict, w: Dict[str, np.ndarray], ids, layers: Optional[int] = None, rows=None,
            layer_outputs: Optional[list] = None, window: Optional[int] = None, rounded: bool = False) -> np.ndarray:
    """Logits [T, vocab] of a whole sequence (crates/coheryn-engine/src/inference.rs:403-561
    applied to every position at once); with ``rows`` only those positions' logits (the final norm
    and the output product run for the rows whose logits are wanted, inference.rs:545-553).
    ``layer_outputs``, a list, receives every layer's output [T, hidden] (the "blk.{i}.output" of
    inference.rs:541-543).  ``window`` (not in the reference's Qwen2) hides keys at p - window and before.

    ``rounded``: the same arithmetic, but everything a part hands to the next (normalised rows,
    q/k/v, rotated q and k, the attention output, the two projections' outputs, the gated
    activation) is rounded to bfloat16 first; residual stream, reductions and logits stay as they
    are.  The distance between this model and the unrounded one is what keeping activations and
    cache in bfloat16 costs by itself, whoever does the arithmetic: the yardstick for a bfloat16
    engine's distance from the unrounded model."""
    rnd = round_bf16 if rounded else None
    T = len(ids)
    positions = np.arange(T)
    x = embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"] if layers is None else layers):
        x = decoder_layer(x, w, f"model.layers.{i}", cfg, positions, window, rnd)
        if layer_outputs is not None:
            layer_outputs.append(x)
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    y = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    if rounded:
        y = round_bf16(y)
    head = w.get("lm_head.weight")
    if head is None:
        head = w["model.embed_tokens.weight"]   # tied (inference.rs:548-552)
    return linear(y, head)


def greedy(cfg: dict, w: Dict[str, np.ndarray], prompt, steps: int):
    """Greedy continuation, recomputing the whole sequence each step; ties go to the
    lowest id (crates/coheryn-engine/src/sampling.rs:160-173)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(np.argmax(forward(cfg, w, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


# ------------------------------------------------------------------------------ sampler
class PlainSampler:
    """The reference's sampler (crates/coheryn-engine/src/sampling.rs:57-224): penalties,
    mask, temperature, top-k, top-p and a SplitMix64 draw, all in float64."""

    MASK = (1 << 64) - 1

    def __init__(self, temperature=0.0, top_k=0, top_p=1.0, seed=0, repetition_penalty=1.0,
                 frequency_penalty=0.0, presence_penalty=0.0):
        self.t, self.k, self.p = float(f32(temperature)), int(top_k), float(f32(top_p))
        self.state = int(seed) & self.MASK
        self.rep = float(f32(repetition_penalty))
        self.freq = float(f32(frequency_penalty))
        self.pres = float(f32(presence_penalty))
        self.counts: Dict[int, int] = {}

    def enabled(self):
        return self.rep != 1.0 or self.freq != 0.0 or self.pres != 0.0

    def observe(self, token: int):
        if self.enabled():
            self.counts[token] = self.counts.get(token, 0) + 1

    def random(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.MASK
        return ((z ^ (z >> 31)) >> 11) / float(1 << 53)

    def adjusted(self, i: int, value) -> float:
        v = float(value)
        c = self.counts.get(i, 0)
        if c:
            v = v * self.rep if v < 0 else v / self.rep
            v -= self.pres + c * self.freq
        return v

    def sample(self, logits, allowed=None) -> int:
        logits = np.asarray(logits, dtype=f32)
        if logits.size == 0 or not np.isfinite(logits).all():
            raise ValueError("empty or non-finite logits")
        ids = [i for i in range(len(logits)) if allowed is None or allowed[i]]
        if not ids:
            raise ValueError("sampling mask permits no token")
        val = {i: self.adjusted(i, logits[i]) for i in ids}
        if self.t == 0.0:
            best = ids[0]
            for i in ids:
                if val[i] > val[best]:
                    best = i
            return best
        ids.sort(key=lambda i: (-val[i], i))
        if 0 < self.k < len(ids):
            ids = ids[:self.k]
        mx = val[ids[0]]
        probs = [float(np.exp((val[i] - mx) / self.t)) for i in ids]
        total = sum(probs)
        cum, n = 0.0, 0
        for pr in probs:
            cum += pr / total
            n += 1
            if cum >= self.p:
                break
        probs = probs[:n]
        threshold = self.random() * sum(probs)
        cum = 0.0
        for i, pr in zip(ids, probs):
            cum += pr
            if threshold < cum:
                return i
        return ids[n - 1]
