"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  Only
the tokens given are run, as one batch, against what earlier steps left in the cache;
logits come back only for the places asked for.  The reference's batched forward takes
exactly one token per lane (crates/coheryn-engine/src/inference/batch.rs:64-116) and
returns logits for every lane; here a lane carries any number of tokens and logits are
computed for the wanted rows alone (the non-output shortcut of
crates/coheryn-engine/src/inference.rs:481-485 taken further).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import StepContext
from ..parts.model import DecoderModel


class OutOfPages(RuntimeError):
    """The cache pool cannot hold the tokens of this step."""


@dataclass
class StepEntry:
    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are wanted


class StepRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager):
        self.model, self.cache = model, cache
        self.device = model.runtime.device
        self.layer_caches = cache.layer_caches()
        self.steps_run = 0

    def _to_device(self, array: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(array)
        if self.device.type == "cuda":
            t = t.pin_memory()
        return t.to(self.device, non_blocking=True)

    def build_context(self, entries: Sequence[StepEntry]):
        """Reserve pages and lay the batch out for the device.  Raises OutOfPages (with
        every reservation of this step undone) when the pool is too small."""
        cache, spec = self.cache, self.model.spec
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request_id!r} brings no token")
            start = cache.length(e.request_id)
            if start + len(e.tokens) > spec.max_positions:
                raise ValueError(f"request {e.request_id!r} would reach position "
                                 f"{start + len(e.tokens)}, beyond the model's {spec.max_positions}")
            for t in e.tokens:
                if not 0 <= int(t) < spec.vocab_size:
                    raise ValueError(f"token id {t} is outside the vocabulary (0..{spec.vocab_size - 1})")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.request_id!r} wants the logits of place {w} "
                                     f"of {len(e.tokens)} tokens")
        done: List[str] = []
        for e in entries:
            if not cache.reserve(e.request_id, e.tokens):
                for rid in done:
                    cache.rollback(rid)
                raise OutOfPages(f"no cache pages left for {len(e.tokens)} more tokens of request "
                                 f"{e.request_id!r} (available per group: {cache.available_pages()})")
            done.append(e.request_id)

        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        starts = [cache.length(e.request_id) for e in entries]
        kv_lens = [s + n for s, n in zip(starts, q_lens)]
        T = sum(q_lens)
        ids = np.empty(T, np.int32); pos = np.empty(T, np.int32); req = np.empty(T, np.int32)
        cu = np.zeros(B + 1, np.int32)
        rows: List[int] = []
        o = 0
        for b, e in enumerate(entries):
            n = q_lens[b]
            ids[o:o + n] = np.asarray(e.tokens, dtype=np.int32)
            pos[o:o + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            req[o:o + n] = b
            rows.extend(o + int(w) for w in e.want)
            o += n
            cu[b + 1] = o
        tables, slots = [], []
        for gi in range(len(cache.groups)):
            lists = [cache.block_table(e.request_id, gi) for e in entries]
            width = max(1, max(len(l) for l in lists))
            bt = np.full((B, width), -1, np.int32)
            for b, l in enumerate(lists):
                bt[b, :len(l)] = l
            tables.append(self._to_device(bt))
            sl = np.concatenate([np.asarray(cache.slot_ids(e.request_id, gi), np.int32) for e in entries])
            slots.append(self._to_device(sl))
        ctx = StepContext(
            num_tokens=T, num_requests=B,
            token_ids=self._to_device(ids), positions=self._to_device(pos),
            token_req=self._to_device(req), cu_q=self._to_device(cu),
            kv_lens=self._to_device(np.asarray(kv_lens, np.int32)),
            block_tables=tables, slots=slots,
            state_slots=self._to_device(np.asarray([cache.state_slot(e.request_id) for e in entries], np.int32)),
            q_lens=q_lens, kv_lens_host=kv_lens, max_q_len=max(q_lens), max_kv_len=max(kv_lens))
        return ctx, self._to_device(np.asarray(rows, np.int32))

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the batch; returns float32 logits ``[wanted, vocab]`` on the device, in the
        order of the entries and of their ``want`` lists."""
        ctx, rows = self.build_context(entries)
        try:
            logits = self.model.forward(ctx, self.layer_caches, rows)
        except Exception:
            for e in entries:
                self.cache.rollback(e.request_id)
            raise
        for e in entries:
            self.cache.commit(e.request_id)
        self.steps_run += 1
        return logits

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input (an id outside the table, non-finite logits)."""
        code = int(self.model.status.item())
        if code:
            self.model.status.zero_()
            raise RuntimeError({1: "a token id was outside the embedding table",
                                2: "non-finite logits"}.get(code, f"device status {code}"))
