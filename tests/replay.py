"""Test harness: drives the engine's step function with scripted steps (the same shape as
bin/trace_run's input) and compares the logits with the plain implementation."""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np
import torch

import plain_qwen2 as plain
from coheryn_ai_studio_b200.cache import CacheManager
from coheryn_ai_studio_b200.engine import StepEntry, StepRunner, load_model, parse_dtype

# Stated tolerances.  float32: the engine differs from the plain implementation only in
# the order of float32 sums.  bfloat16: weights are identical (the folders hold bfloat16
# values); activations and cache are rounded to 8 bits of mantissa at every part, so the
# bound is relative to the spread of the logits.
TOL_F32 = 1e-4


def tol_bf16(ref: np.ndarray) -> float:
    return 0.04 * max(1.0, float(np.abs(ref).max()))


class Replay:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16,
                 max_requests: int = 8, model=None):
        self.dtype = dtype
        self.model = model if model is not None else load_model(model_dir, dtype)[1]
        self.cache = CacheManager(self.model.cache_requirements(),
                                  [e.cache_from for e in self.model.spec.schedule],
                                  parse_dtype(dtype), torch.device("cuda:0"), page_size=page_size,
                                  num_pages=-(-max_tokens // page_size), max_requests=max_requests,
                                  prefix_reuse=False)
        self.runner = StepRunner(self.model, self.cache)
        self.positions: Dict[str, int] = {}
        self.rows: Dict[Tuple[str, int], np.ndarray] = {}
        self.pages_seen: Dict[int, int] = {}

    def step(self, entries: List[Tuple[str, List[int], List[int]]], end=()):
        batch = []
        for rid, toks, want in entries:
            if rid not in self.cache.requests:
                assert self.cache.admit(rid) is not None
                self.positions[rid] = 0
            batch.append(StepEntry(rid, toks, want))
        logits = self.runner.step(batch).cpu().numpy()
        self.runner.check_status()
        self.cache.check()
        for rid, _, _ in entries:
            for p in self.cache.block_table(rid, 0):
                if p >= 0:
                    self.pages_seen[p] = self.pages_seen.get(p, 0)
        i = 0
        for rid, toks, want in entries:
            for w in want:
                self.rows[(rid, self.positions[rid] + w)] = logits[i]
                i += 1
            self.positions[rid] += len(toks)
        assert i == logits.shape[0]
        for rid in end:
            self.cache.free(rid)
            del self.positions[rid]
        self.cache.check()


_plain_cache: Dict[Tuple[str, Tuple[int, ...]], np.ndarray] = {}


def plain_logits(model_dir: str, tokens: List[int]) -> np.ndarray:
    key = (model_dir, tuple(tokens))
    if key not in _plain_cache:
        cfg, w = plain.read_model(model_dir)
        _plain_cache[key] = plain.forward(cfg, w, tokens)
    return _plain_cache[key]


def compare(replay: Replay, model_dir: str, sequences: Dict[str, List[int]], label: str = ""):
    """Every recorded row against the plain implementation of the request's whole
    sequence.  Returns the largest difference seen."""
    worst = 0.0
    for (rid, pos), row in sorted(replay.rows.items()):
        ref = plain_logits(model_dir, sequences[rid])[pos]
        diff = float(np.abs(row - ref).max())
        worst = max(worst, diff)
        if replay.dtype == "float32":
            assert diff <= TOL_F32, f"{label} {rid}@{pos}: |d|={diff:.3e} > {TOL_F32}"
            assert int(row.argmax()) == int(ref.argmax()) or np.sort(ref)[-1] - np.sort(ref)[-2] < 2 * TOL_F32, \
                f"{label} {rid}@{pos}: argmax differs"
        else:
            t = tol_bf16(ref)
            assert diff <= t, f"{label} {rid}@{pos}: |d|={diff:.3e} > {t:.3e}"
    return worst
