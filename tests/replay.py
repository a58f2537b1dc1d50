"""Test harness: drives the engine's step function with scripted steps (the same shape as
bin/trace_run's input) and compares the logits with the plain implementation."""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np
import torch

import plain_qwen2 as plain
from coheryn_ai_studio_b200.cache import CacheManager
from coheryn_ai_studio_b200.engine import StepEntry, StepRunner, load_model, parse_dtype

# Stated tolerances.
# float32: the engine differs from the plain implementation only in the order of float32 sums.
# bfloat16: the weights are identical (the folders hold bfloat16 values), but activations and cache
# are rounded to 8 bits of mantissa between the parts.  What that costs by itself is measured, row by
# row, on the plain implementation: plain.forward(rounded=True) rounds at the same places and does
# everything else as before.  A bfloat16 engine may be as far from the unrounded plain row as a
# small factor times that distance (its rounding errors are other draws of the same noise, and it
# rounds in a few more places, such as the probabilities), measured both as the root mean square over
# the row and as the largest error in it.  ``assert_bound_sees_a_wrong_token`` checks on the plain model that ONE wrong
# token among the keys moves a row out of this bound, so it cannot grow until it swallows such a
# fault without a test failing.
TOL_F32 = 1e-4
BF16_RMS_FACTOR = 2.0       # root mean square of a row's error: the sharp criterion (a stable statistic)
BF16_MAX_FACTOR = 3.0       # largest error of a row: looser, the largest of hundreds of draws scatters
BF16_MIN_SIGMAS = 0.02      # of the row's spread, for the largest error; a quarter of it for the rms


def tol_bf16(ref_row: np.ndarray, rounded_row: np.ndarray) -> float:
    """Bound on the largest error of a row."""
    sigma = float(np.std(ref_row.astype(np.float64)))
    return BF16_MAX_FACTOR * max(BF16_MIN_SIGMAS * sigma, float(np.abs(rounded_row - ref_row).max()))


def tol_bf16_rms(ref_row: np.ndarray, rounded_row: np.ndarray) -> float:
    """Bound on the root mean square error of a row."""
    sigma = float(np.std(ref_row.astype(np.float64)))
    d = (rounded_row - ref_row).astype(np.float64)
    return BF16_RMS_FACTOR * max(0.25 * BF16_MIN_SIGMAS * sigma, float(np.sqrt(np.mean(d * d))))


LARGEST_EXCESS = {"value": 0.0, "rows": 0}      # over a test session, reported by conftest.py


def bf16_excess(row: np.ndarray, ref_row: np.ndarray, rounded_row: np.ndarray, record: bool = False) -> float:
    """How far a bfloat16 row is from the plain row, in units of what is allowed (<= 1 passes): the
    larger of rms error / rms bound and largest error / bound on the largest."""
    d = (row - ref_row).astype(np.float64)
    excess = max(float(np.sqrt(np.mean(d * d))) / tol_bf16_rms(ref_row, rounded_row),
                 float(np.abs(d).max()) / tol_bf16(ref_row, rounded_row))
    if record:                                   # rows of the engine (not the deliberately wrong rows of the self-checks)
        LARGEST_EXCESS["value"] = max(LARGEST_EXCESS["value"], excess)
        LARGEST_EXCESS["rows"] += 1
    return excess


def tol_bf16_spread(row: np.ndarray, sigmas: float = 0.04) -> float:
    """For comparisons that have no rounded twin at hand (two runs of the engine against each other;
    a toy model whose plain restatement lives in its test): a share of the row's spread."""
    return sigmas * float(np.std(row.astype(np.float64)))


def assert_bound_sees_a_wrong_token(model_dir: str, tokens: List[int], places=(0, 1, 2, None)) -> float:
    """Change one token of the sequence (so one key and one value of every layer are wrong for
    all later rows) and check on the plain model that the LAST row then moves by more than the
    bfloat16 bound, for a change at the start and in the middle of the sequence.  Returns the
    smallest move seen, in units of the bound."""
    cfg, w = plain.read_model(model_dir)
    last = len(tokens) - 1
    ref = plain_logits(model_dir, tokens)[last]
    twin = plain_logits(model_dir, tokens, rounded=True)[last]
    worst = float("inf")
    for place in places:
        j = len(tokens) // 2 if place is None else place
        if j >= len(tokens) - 1:
            continue
        changed = list(tokens)
        changed[j] = (changed[j] + 1) % cfg["vocab_size"]
        excess = bf16_excess(plain.forward(cfg, w, changed, rows=[last])[0], ref, twin)
        assert excess > 1.25, (f"a wrong token at place {j} of {len(tokens)} moves the last row by {excess:.2f} of "
                               "what the bfloat16 bound allows: it would not be seen")
        worst = min(worst, excess)
    return worst


class Replay:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16,
                 max_requests: int = 8, model=None, use_graphs: bool = False, prefix_reuse: bool = False,
                 layer_outputs: bool = False):
        self.dtype = dtype
        self.model = model if model is not None else load_model(model_dir, dtype)[1]
        self.cache = CacheManager(self.model.cache_requirements(),
                                  [e.cache_from for e in self.model.spec.schedule],
                                  parse_dtype(dtype), torch.device("cuda:0"), page_size=page_size,
                                  num_pages=-(-max_tokens // page_size), max_requests=max_requests,
                                  prefix_reuse=prefix_reuse)
        # The pool starts full of noise instead of zeros: a kernel that reads a slot which no step of
        # the request has written (a stale page, a key fetched before it was stored) then shows.
        for g in self.cache.groups:
            g.tensor.normal_(0.0, 8.0)
        self.runner = StepRunner(self.model, self.cache, use_graphs=use_graphs, graph_max_kv_len=max_tokens)
        self.positions: Dict[str, int] = {}
        self.rows: Dict[Tuple[str, int], np.ndarray] = {}
        self.pages_seen: Dict[int, int] = {}
        self.reused: Dict[str, int] = {}
        # (request, position) -> [schedule entries, hidden]: every layer's output, when asked for
        self.layers: Dict[Tuple[str, int], np.ndarray] = {}
        self.layer_outputs = layer_outputs

    def admit(self, rid: str, prompt: List[int]) -> int:
        """Admit a request with its whole prompt known, so that leading pages another request
        filled are mapped instead of computed; returns how many tokens that saves.  The caller
        then feeds the prompt from that place on."""
        reused = self.cache.admit(rid, prompt)
        assert reused is not None
        self.positions[rid] = reused
        self.reused[rid] = reused
        return reused

    def step(self, entries: List[Tuple[str, List[int], List[int]]], end=()):
        batch = []
        for rid, toks, want in entries:
            if rid not in self.cache.requests:
                assert self.cache.admit(rid) is not None
                self.positions[rid] = 0
            batch.append(StepEntry(rid, toks, want))
        seen = []
        if self.layer_outputs:
            self.model.layer_observer = lambda entry, x: seen.append(x.float().cpu().numpy())
        try:
            logits = self.runner.step(batch).cpu().numpy()
        finally:
            self.model.layer_observer = None
        if seen:
            stack = np.stack(seen)                       # [entries, T, H]
            o = 0
            for rid, toks, _ in entries:
                for t in range(len(toks)):
                    self.layers[(rid, self.positions[rid] + t)] = stack[:, o + t]
                o += len(toks)
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


_plain_cache: Dict[Tuple[str, Tuple[int, ...], bool], np.ndarray] = {}


def plain_logits(model_dir: str, tokens: List[int], rounded: bool = False) -> np.ndarray:
    """Logits of the whole sequence by the plain implementation (``rounded``: its twin that rounds
    what passes between parts to bfloat16)."""
    key = (model_dir, tuple(tokens), rounded)
    if key not in _plain_cache:
        cfg, w = plain.read_model(model_dir)
        _plain_cache[key] = plain.forward(cfg, w, tokens, rounded=rounded)
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
            excess = bf16_excess(row, ref, plain_logits(model_dir, sequences[rid], rounded=True)[pos], record=True)
            assert excess <= 1.0, f"{label} {rid}@{pos}: {excess:.2f} of the bfloat16 bound (largest |d| = {diff:.3e})"
    return worst


def assert_greedy_follows_plain(model_dir: str, prompt: List[int], tokens: List[int], dtype: str, label: str = ""):
    """Every generated token, given the tokens before it, is the plain implementation's choice: the
    first maximum of the plain logits, or, in bfloat16, a token whose plain logit lies within twice
    the bound of that maximum (a near-tie that rounding may decide either way).  The walk follows
    the ENGINE's tokens, so every one of them is checked, also after a near-tie."""
    cfg, w = plain.read_model(model_dir)
    ids = list(prompt)
    for k, tok in enumerate(tokens):
        ref = plain.forward(cfg, w, ids, rows=[len(ids) - 1])[0]
        best = int(np.argmax(ref))
        if tok != best:
            gap = float(ref[best] - ref[tok])
            assert dtype != "float32" or gap < 2 * TOL_F32, f"{label} token {k}: {tok} is not the plain choice {best}"
            bound = 2 * tol_bf16(ref, plain.forward(cfg, w, ids, rows=[len(ids) - 1], rounded=True)[0])
            assert gap <= bound, (f"{label} token {k}: {tok} lies {gap:.4f} below the plain choice {best}, "
                                  f"more than rounding explains ({bound:.4f})")
        ids.append(tok)
