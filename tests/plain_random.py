"""The seeded random weights of the engine's random-weights mode, restated in numpy for the
plain implementation: value(seed, tensor name, element index), so that the plain model can
make the very weights a model on the device holds, for the whole tensor or for a few rows.

    key   = seed XOR fnv1a64(name)
    draw(n) = n-th output of SplitMix64 from state key (constants of
              crates/coheryn-engine/src/sampling.rs:123-130)
    u1 = ((draw(2i+1) >> 11) + 1) / 2^53,  u2 = (draw(2i+2) >> 11) / 2^53
    value(i) = float32(mean + deviation * sqrt(-2 ln u1) * cos(2 pi u2))

ln and cos are evaluated with float64 additions, multiplications and divisions in a fixed
order (numpy rounds after every operation), so the result does not depend on a maths
library; the engine's C++ and CUDA versions do the same operations in the same order.
This file shares no code with them.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Optional, Sequence

import numpy as np

MASK = (1 << 64) - 1
GAMMA, C1, C2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & MASK
    return h


def tensor_key(seed: int, name: str) -> int:
    return (int(seed) & MASK) ^ fnv1a64(name)


def _draw(key: int, n: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = np.uint64(key) + n * np.uint64(GAMMA)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(C1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(C2)
        return z ^ (z >> np.uint64(31))


def _ln_unit(k: np.ndarray) -> np.ndarray:
    """ln(k / 2^53) for integers 1 <= k <= 2^53."""
    one = k >> np.uint64(53) != 0
    k = np.where(one, np.uint64(1) << np.uint64(52), k)
    # position of the leading one, by halving steps (integers only)
    lead = np.zeros(k.shape, np.int64)
    rest = k.copy()
    for shift in (32, 16, 8, 4, 2, 1):
        big = rest >> np.uint64(shift) != 0
        lead += np.where(big, shift, 0)
        rest = np.where(big, rest >> np.uint64(shift), rest)
    m = (k << (np.uint64(52) - lead.astype(np.uint64))).astype(np.float64) * (1.0 / 4503599627370496.0)
    e = lead - 53
    up = m > 1.4142135623730951
    m = np.where(up, m * 0.5, m)
    e = np.where(up, e + 1, e)
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = np.full(k.shape, 1.0 / 23.0)
    for d in (21.0, 19.0, 17.0, 15.0, 13.0, 11.0, 9.0, 7.0, 5.0, 3.0):
        p = p * s2 + 1.0 / d
    p = p * s2 + 1.0
    ln_m = (2.0 * s) * p
    out = e.astype(np.float64) * 0.6931471805599453 + ln_m
    return np.where(one, 0.0, out)


def _cos_turn(j: np.ndarray) -> np.ndarray:
    """cos(2 pi j / 2^53) for integers 0 <= j < 2^53."""
    quarter = (j >> np.uint64(51)).astype(np.int64)
    g = (j & np.uint64((1 << 51) - 1)).astype(np.float64) * (1.0 / 2251799813685248.0)
    x = (g + -0.5) * 1.5707963267948966
    x2 = x * x
    c = np.full(j.shape, 1.0 / 6402373705728000.0)
    for f in (-1.0 / 20922789888000.0, 1.0 / 87178291200.0, -1.0 / 479001600.0, 1.0 / 3628800.0,
              -1.0 / 40320.0, 1.0 / 720.0, -1.0 / 24.0, 0.5):
        c = c * x2 + f
    c = (c * x2) * -1.0 + 1.0
    s = np.full(j.shape, 1.0 / 121645100408832000.0)
    for f in (-1.0 / 355687428096000.0, 1.0 / 1307674368000.0, -1.0 / 6227020800.0, 1.0 / 39916800.0,
              -1.0 / 362880.0, 1.0 / 5040.0, -1.0 / 120.0, 1.0 / 6.0):
        s = s * x2 + f
    s = (s * x2) * -1.0 + 1.0
    s = s * x
    r = 0.7071067811865476
    cos_q = (c + s * -1.0) * r
    sin_q = (s + c) * r
    return np.select([quarter == 0, quarter == 1, quarter == 2], [cos_q, sin_q * -1.0, cos_q * -1.0], sin_q)


def values(key: int, index: np.ndarray, mean: float, deviation: float) -> np.ndarray:
    """float32 values of the elements ``index`` (any shape, uint64) of the tensor with ``key``."""
    index = np.asarray(index, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = _draw(key, np.uint64(2) * index + np.uint64(1))
        b = _draw(key, np.uint64(2) * index + np.uint64(2))
    ln_u = _ln_unit((a >> np.uint64(11)) + np.uint64(1))
    radius = np.sqrt(-2.0 * ln_u)
    z = radius * _cos_turn(b >> np.uint64(11))
    return (mean + deviation * z).astype(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16 (ties to even), kept as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def tensor(seed: int, name: str, shape: Sequence[int], mean: float, deviation: float,
           rows: Optional[Sequence[int]] = None, bf16: bool = False, threads: int = 16) -> np.ndarray:
    """The tensor ``name`` of a model made from ``seed`` (or only its rows ``rows``), as float32;
    with ``bf16`` every value is rounded to bfloat16 first, as the stored weights are."""
    key = tensor_key(seed, name)
    shape = tuple(int(d) for d in shape)
    inner = int(np.prod(shape[1:])) if len(shape) > 1 else 1
    row_ids = np.arange(shape[0], dtype=np.uint64) if rows is None else np.asarray(rows, dtype=np.uint64)

    def chunk(part: np.ndarray) -> np.ndarray:
        idx = part[:, None] * np.uint64(inner) + np.arange(inner, dtype=np.uint64)[None, :]
        v = values(key, idx, mean, deviation)
        return round_bf16(v) if bf16 else v

    per = max(1, (1 << 19) // max(inner, 1))
    parts = [row_ids[i:i + per] for i in range(0, len(row_ids), per)]
    if len(parts) > 1 and threads > 1:
        with ThreadPoolExecutor(threads) as ex:
            done = list(ex.map(chunk, parts))
    else:
        done = [chunk(p) for p in parts]
    out = np.concatenate(done, axis=0) if done else np.zeros((0, inner), np.float32)
    return out.reshape((len(row_ids),) + shape[1:])
