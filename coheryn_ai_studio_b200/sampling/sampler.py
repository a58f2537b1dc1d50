"""Sampling in the reference's manner (crates/coheryn-engine/src/sampling.rs, profile
"coheryn-sampling-v2"): temperature 0 is greedy with ties to the lowest id; otherwise
candidates are ranked by (value descending, id ascending), top-k keeps the first k, top-p
the shortest prefix whose normalised mass reaches it, and one SplitMix64 draw per sampled
token picks the candidate whose cumulative mass first exceeds ``u * kept mass``.
Penalties over the ids seen so far (prompt and generated) come first: for a seen id,
``v = v * rep if v < 0 else v / rep``, then ``v -= presence + count * frequency``.

The draw is made on the host (one 64-bit state per request, advanced only when a token is
sampled); selection runs on the device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0

    def validate(self, vocab_size: Optional[int] = None) -> None:
        """Ranges of sampling.rs:75-84 and 38-52."""
        t, p = self.temperature, self.top_p
        if not (math.isfinite(t) and 0.0 <= t <= 2.0 and math.isfinite(p) and 0.0 < p <= 1.0):
            raise ValueError("temperature must be finite in [0,2]; top_p must be in (0,1]")
        if not (math.isfinite(self.repetition_penalty) and 0.01 <= self.repetition_penalty <= 10.0
                and math.isfinite(self.frequency_penalty) and -2.0 <= self.frequency_penalty <= 2.0
                and math.isfinite(self.presence_penalty) and -2.0 <= self.presence_penalty <= 2.0):
            raise ValueError("repetition_penalty must be in [0.01,10]; frequency/presence penalties "
                             "must be in [-2,2]; all must be finite")
        if self.top_k < 0 or (vocab_size is not None and self.top_k > vocab_size):
            raise ValueError("top_k exceeds model vocabulary")
        if not 0 <= self.seed <= _MASK:
            raise ValueError("seed must fit 64 unsigned bits")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def penalised(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0)


class SplitMix64:
    """sampling.rs:123-130."""

    def __init__(self, seed: int):
        self.state = int(seed) & _MASK

    def random(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return ((z ^ (z >> 31)) >> 11) / float(1 << 53)


class RequestSampler:
    """Per-request sampling state: the random stream and the counts of seen ids."""

    def __init__(self, params: SamplingParams, history: Sequence[int] = ()):
        self.params = params
        self.rng = SplitMix64(params.seed)
        self.counts: Dict[int, int] = {}
        if params.penalised:
            for t in history:
                self.observe(t)

    def observe(self, token: int) -> None:
        if self.params.penalised:
            self.counts[token] = self.counts.get(token, 0) + 1


class DeviceSampler:
    """Picks one token per logits row on the device."""

    def __init__(self, device):
        self.device = device
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def _dev(self, array: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(array)
        if self.device.type == "cuda":
            t = t.pin_memory()
        return t.to(self.device, non_blocking=True)

    def sample(self, logits: torch.Tensor, samplers: Sequence[RequestSampler]) -> List[int]:
        """logits: float32 [R, V] (modified in place when penalties apply).  Returns the
        chosen ids; advances each sampled request's random stream by one draw and records
        the chosen id in its counts."""
        return self.finish(self.launch(logits, samplers))

    def launch(self, logits: torch.Tensor, samplers: Sequence[RequestSampler], extra_status=()) -> "PendingSample":
        """Start the selection and the copy of its result to pinned host memory; nothing waits.
        ``extra_status``: further device status words (int32[1]) copied along.  The chosen ids
        stay on the device in ``PendingSample.ids`` (the next step may read them there)."""
        R = logits.shape[0]
        assert R == len(samplers)
        if R == 0:
            return PendingSample(None, None, None, list(samplers), [])
        rows, ids, counts, rep, freq, pres = [], [], [], [], [], []
        for r, s in enumerate(samplers):
            if s.params.penalised and s.counts:
                for tok, c in s.counts.items():
                    rows.append(r); ids.append(tok); counts.append(c)
                    rep.append(s.params.repetition_penalty)
                    freq.append(s.params.frequency_penalty); pres.append(s.params.presence_penalty)
        if rows:
            ops.apply_penalties(logits, self._dev(np.asarray(rows, np.int32)),
                                self._dev(np.asarray(ids, np.int32)), self._dev(np.asarray(counts, np.int32)),
                                self._dev(np.asarray(rep, np.float32)), self._dev(np.asarray(freq, np.float32)),
                                self._dev(np.asarray(pres, np.float32)))
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        hot = [r for r, s in enumerate(samplers) if not s.params.greedy]
        if len(hot) < R:
            ops.argmax(logits, out, self.status)
        if hot:
            hot_rows = self._dev(np.asarray(hot, np.int32))
            sub = logits if len(hot) == R else ops.gather_rows(logits, hot_rows)
            temp = np.asarray([samplers[r].params.temperature for r in hot], np.float32)
            topk = np.asarray([samplers[r].params.top_k for r in hot], np.int32)
            topp = np.asarray([samplers[r].params.top_p for r in hot], np.float32)
            u = np.asarray([samplers[r].rng.random() for r in hot], np.float64)
            picked = torch.empty(len(hot), dtype=torch.int32, device=self.device)
            ops.sample(sub, self._dev(temp), self._dev(topk), self._dev(topp), self._dev(u), picked, self.status)
            if len(hot) == R:
                out = picked
            else:
                ops.scatter_words(picked, hot_rows, out)
        words = [self.status] + list(extra_status)
        host = self._pinned(R + len(words))
        host[:R].copy_(out, non_blocking=True)
        for i, w in enumerate(words):
            host[R + i:R + i + 1].copy_(w, non_blocking=True)
        event = torch.cuda.Event() if self.device.type == "cuda" else None
        if event is not None:
            event.record()
        return PendingSample(out, host, event, list(samplers), words)

    def _pinned(self, n: int) -> torch.Tensor:
        """One of a few pinned buffers handed out in turn (at most two selections are in
        flight at a time)."""
        if self.device.type != "cuda":
            return torch.empty(n, dtype=torch.int32)
        self._turn = (getattr(self, "_turn", -1) + 1) % 4
        pool = self.__dict__.setdefault("_pool", [None] * 4)
        if pool[self._turn] is None or pool[self._turn].numel() < n:
            pool[self._turn] = torch.empty(max(n, 256), dtype=torch.int32).pin_memory()
        return pool[self._turn][:n]

    def finish(self, pending: "PendingSample") -> List[int]:
        """Wait for a launched selection (and for nothing launched after it); returns the ids."""
        if pending.host is None:
            return []
        if pending.event is not None:
            pending.event.synchronize()
        values = pending.host.tolist()
        R = len(pending.samplers)
        chosen, status = values[:R], values[R:]
        if any(status):
            for w in pending.words:
                w.zero_()
            if status[0]:
                raise RuntimeError("empty or non-finite logits")
            raise RuntimeError(ops.describe_status(max(status[1:])))
        for s, tok in zip(pending.samplers, chosen):
            s.observe(tok)
        return chosen


class PendingSample:
    """A selection in flight: ids on the device, their pinned host copy and its event."""

    def __init__(self, ids, host, event, samplers, words):
        self.ids, self.host, self.event, self.samplers, self.words = ids, host, event, samplers, words
