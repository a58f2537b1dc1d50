"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  Only
the tokens given are run, as one batch, against what earlier steps left in the cache;
logits come back only for the places asked for.  The reference's batched forward takes
exactly one token per lane (crates/coheryn-engine/src/inference/batch.rs:64-116) and
returns logits for every lane; here a lane carries any number of tokens and logits are
computed for the wanted rows alone.  When at most half of the rows are wanted, the last
entry of the schedule also runs its attention and feed-forward for the wanted rows only,
after it has written the keys and values of all of them (the non-output shortcut of
crates/coheryn-engine/src/inference.rs:481-485).

Steps in which every request brings exactly one token and wants its logits (decoding) can
be replayed from a CUDA graph: the launch sequence is captured once per batch width over
static index buffers, and a step then costs one host-to-device copy and one graph launch.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
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


@dataclass
class _Layout:
    """A batch as host arrays (all int32)."""
    B: int
    T: int
    ids: np.ndarray
    pos: np.ndarray
    req: np.ndarray
    cu: np.ndarray
    kv_lens: np.ndarray
    state_slots: np.ndarray
    rows: np.ndarray
    tables: List[List[np.ndarray]]    # per group, per request: pages
    slots: List[np.ndarray]           # per group: [T]
    q_lens: List[int]
    serials: List[int] = field(default_factory=list)     # per request: the number of its admission


class _DecodeGraph:
    """The captured launch sequence of a decode step for one batch width.  A batch of fewer
    rows than the width is padded: the extra rows are one-token requests at position 0 whose
    only page is the cache's spare page, and their logits are dropped."""

    STAGES = 3

    def __init__(self, runner: "StepRunner", B: int):
        self.B = B
        self.used = B            # rows of the last fill that were real
        self.spare_page = runner.cache.spare_page
        self.page_size = runner.cache.page_size
        groups = len(runner.cache.groups)
        self.width = runner.graph_table_width
        sizes = [("ids", B), ("pos", B), ("req", B), ("cu", B + 1), ("kv_lens", B), ("state_slots", B),
                 ("rows", B)]
        for g in range(groups):
            sizes += [(f"table{g}", B * self.width), (f"slots{g}", B)]
        total = sum(n for _, n in sizes)
        # The batch is kept in an ordinary host array (rows that stay get only what they gained)
        # and leaves through one of a few pinned staging buffers handed out in turn: an asynchronous
        # copy reads its pinned source when the device gets to it, so a buffer is written again only
        # after the copy that last used it has completed (its event), however far the host runs ahead.
        self.master = np.zeros(total, dtype=np.int32)
        self.stages = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(self.STAGES)]
        self.stage_events: List[Optional[torch.cuda.Event]] = [None] * self.STAGES
        self.turn = 0
        self.dev = torch.zeros(total, dtype=torch.int32, device=runner.device)
        self.nbytes = total * 4
        self.h: Dict[str, np.ndarray] = {}
        self.d: Dict[str, torch.Tensor] = {}
        o = 0
        for name, n in sizes:
            self.h[name] = self.master[o:o + n]
            self.d[name] = self.dev[o:o + n]
            o += n
        self.ctx = StepContext(
            num_tokens=B, num_requests=B, token_ids=self.d["ids"], positions=self.d["pos"],
            token_req=self.d["req"], cu_q=self.d["cu"], kv_lens=self.d["kv_lens"],
            block_tables=[self.d[f"table{g}"].view(B, self.width) for g in range(groups)],
            slots=[self.d[f"slots{g}"] for g in range(groups)], state_slots=self.d["state_slots"],
            q_lens=[1] * B, kv_lens_host=[], max_q_len=1, max_kv_len=runner.graph_max_kv_len)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0
        self.bound = [[(None, 0)] * B for _ in range(groups)]     # per group and row: (request, pages written)
        self.windowed = [g.need.window is not None for g in runner.cache.groups]
        self._pad(0)

    def _pad(self, first: int) -> None:
        """Rows first.. of the host buffer become padding rows."""
        h, B = self.h, self.B
        ar = np.arange(B + 1, dtype=np.int32)
        h["ids"][first:] = 0; h["pos"][first:] = 0; h["req"][first:] = ar[first:B]; h["cu"][:] = ar
        h["kv_lens"][first:] = 1; h["state_slots"][first:] = 0; h["rows"][:] = ar[:B]
        for g in range(len(self.bound)):
            tab = h[f"table{g}"].reshape(B, self.width)
            tab[first:, 0] = self.spare_page
            h[f"slots{g}"][first:] = self.spare_page * self.page_size
            for b in range(first, B):
                self.bound[g][b] = (None, 0)

    def fill(self, lay: _Layout, serials: Sequence[int]) -> None:
        """Write the batch into the pinned buffer and copy it to the device.  A row whose
        request (the same admission: ``serials``) sat there in the last step too only gets the
        pages it has gained since: block tables grow at the end and keep what they held.  (A window that
        gives pages back marks them -1 in place: such rows are written whole.)"""
        h, n_rows = self.h, lay.B
        if n_rows < self.used:       # rows that held requests in the last step are padding now
            self._pad(n_rows)
        self.used = n_rows
        h["ids"][:n_rows] = lay.ids; h["pos"][:n_rows] = lay.pos; h["req"][:n_rows] = lay.req
        h["kv_lens"][:n_rows] = lay.kv_lens; h["state_slots"][:n_rows] = lay.state_slots
        for g, lists in enumerate(lay.tables):
            tab = h[f"table{g}"].reshape(self.B, self.width)
            known = self.bound[g]
            for b, pages in enumerate(lists):
                n = len(pages)
                rid, have = known[b]
                if rid == serials[b] and have <= n and not self.windowed[g]:
                    if have < n:
                        tab[b, have:n] = pages[have:]
                else:
                    tab[b, :n] = pages
                known[b] = (serials[b], n)
            h[f"slots{g}"][:n_rows] = lay.slots[g]
        i = self.turn
        self.turn = (i + 1) % self.STAGES
        if self.stage_events[i] is not None:
            self.stage_events[i].synchronize()       # the copy that last read this buffer is done
        self.stages[i].numpy()[:] = self.master
        self.dev.copy_(self.stages[i], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.stage_events[i] = event

    def forget_rows(self) -> None:
        self.bound = [[(None, 0)] * self.B for _ in self.bound]

    def run(self, runner: "StepRunner") -> torch.Tensor:
        if self.graph is None:
            # The warm-up runs the step for real (it loads libraries and sets kernel attributes outside
            # the capture).  Keys and values land in the same slots every time, but a mixer with state
            # of its own would advance it once per run: that state is put back before the replay.
            states = runner.cache.state_tensors()
            side = torch.cuda.Stream(device=runner.device)
            side.wait_stream(torch.cuda.current_stream(runner.device))
            with torch.cuda.stream(side):
                kept = [t.clone() for t in states]
                for _ in range(2):
                    runner.model.forward(self.ctx, runner.layer_caches, self.d["rows"])
                for t, k in zip(states, kept):
                    t.copy_(k)
            torch.cuda.current_stream(runner.device).wait_stream(side)
            before = ops.total_launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.logits = runner.model.forward(self.ctx, runner.layer_caches, self.d["rows"])
            self.launches = ops.total_launch_count() - before
            self.graph = graph
        self.graph.replay()
        runner.graph_launches += self.launches
        return self.logits[:self.used]


class StepRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, use_graphs: bool = False,
                 graph_max_kv_len: Optional[int] = None):
        """``use_graphs`` replays decode steps from CUDA graphs; ``graph_max_kv_len`` bounds
        the length a request can reach while graphs are used (default: the model's
        positions)."""
        self.model, self.cache = model, cache
        self.device = model.runtime.device
        self.layer_caches = cache.layer_caches()
        self.steps_run = 0
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and model.capturable
        self.graph_max_kv_len = int(graph_max_kv_len or model.spec.max_positions)
        self.graph_table_width = max(1, -(-self.graph_max_kv_len // cache.page_size))
        self._graphs: Dict[int, _DecodeGraph] = {}
        # Steps that want at most half of their rows run the last entry of the schedule for the
        # wanted rows only (COHERYN_TAIL=0 in the environment switches it off).
        self.tail_shortcut = os.environ.get("COHERYN_TAIL", "1") != "0"
        self.graph_launches = 0       # kernel launches replayed from graphs
        self.h2d_bytes = 0            # bytes copied to the device by the last step

    def _to_device(self, array: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(array)
        self.h2d_bytes += array.nbytes
        if self.device.type == "cuda":
            t = t.pin_memory()
        return t.to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ host side
    def _check(self, entries: Sequence[StepEntry]) -> None:
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

    def _reserve(self, entries: Sequence[StepEntry]) -> None:
        done: List[str] = []
        for e in entries:
            if not self.cache.reserve(e.request_id, e.tokens):
                for rid in done:
                    self.cache.rollback(rid)
                raise OutOfPages(f"no cache pages left for {len(e.tokens)} more tokens of request "
                                 f"{e.request_id!r} (available per group: {self.cache.available_pages()})")
            done.append(e.request_id)

    def _layout(self, entries: Sequence[StepEntry]) -> _Layout:
        """The step's arrays from the native book (positions, request of each token, slots, offsets,
        lengths, state slots, admission serials) and the entries (ids, wanted rows)."""
        cache = self.cache
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        groups = len(cache.groups)
        keys = (ctypes.c_char_p * B)(*[str(e.request_id).encode() for e in entries])
        pos = np.empty(T, np.int32); req = np.empty(T, np.int32)
        slots = np.empty(max(groups, 1) * T, np.int32)
        cu = np.empty(B + 1, np.int32); kv_lens = np.empty(B, np.int32); state_slots = np.empty(B, np.int32)
        serials = np.empty(B, np.int64)
        as_int = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
        got = cache._lib.coheryn_book_layout(cache.book_handle, B, keys, as_int(pos), as_int(req), as_int(slots), T, as_int(cu),
                                             as_int(kv_lens), as_int(state_slots),
                                             serials.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong)))
        if got != T:
            raise RuntimeError(f"the cache book laid out {got} tokens where the step brings {T}")
        if T == B:
            ids = np.asarray([e.tokens[0] for e in entries], np.int32)
            rows = [b for b, e in enumerate(entries) for _ in e.want]
        else:
            ids = np.empty(T, np.int32)
            rows = []
            for b, e in enumerate(entries):
                o = int(cu[b])
                ids[o:o + q_lens[b]] = np.asarray(e.tokens, dtype=np.int32)
                rows.extend(o + int(w) for w in e.want)
        lay = _Layout(
            B=B, T=T, ids=ids, pos=pos, req=req, cu=cu, kv_lens=kv_lens, state_slots=state_slots,
            rows=np.asarray(rows, np.int32),
            tables=[self._tables(keys, B, g, int(kv_lens.max())) for g in range(groups)],
            slots=[slots[g * T:(g + 1) * T] for g in range(groups)], q_lens=q_lens)
        lay.serials = serials.tolist()
        return lay

    def _tables(self, keys, B: int, group: int, max_len: int) -> List[np.ndarray]:
        """The block tables of the step's requests for one group, one native call: per request a row
        of page ids (-1 where a window has given the page back)."""
        cache = self.cache
        width = max(1, -(-max_len // cache.page_size))
        as_int = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
        while True:
            out, lens = np.empty((B, width), np.int32), np.empty(B, np.int32)
            longest = cache._lib.coheryn_book_tables(cache.book_handle, B, keys, group, as_int(out), width, as_int(lens))
            if longest < 0:
                raise RuntimeError("the cache book does not know a request of the step")
            if longest <= width:
                return [out[b, :lens[b]] for b in range(B)]
            width = longest

    def _context(self, lay: _Layout):
        tables, host_tables = [], []
        for lists in lay.tables:
            width = max(1, max(len(l) for l in lists))
            bt = np.full((lay.B, width), -1, np.int32)
            for b, l in enumerate(lists):
                bt[b, :len(l)] = l
            host_tables.append(bt)
            tables.append(self._to_device(bt))
        kv = lay.kv_lens.tolist()
        ctx = StepContext(
            num_tokens=lay.T, num_requests=lay.B, token_ids=self._to_device(lay.ids),
            positions=self._to_device(lay.pos), token_req=self._to_device(lay.req),
            cu_q=self._to_device(lay.cu), kv_lens=self._to_device(lay.kv_lens), block_tables=tables,
            slots=[self._to_device(s) for s in lay.slots], state_slots=self._to_device(lay.state_slots),
            q_lens=lay.q_lens, kv_lens_host=kv, max_q_len=max(lay.q_lens), max_kv_len=max(kv))
        rows = self._to_device(lay.rows)
        R = len(lay.rows)
        if self.tail_shortcut and 2 * R <= lay.T:
            # Few rows are wanted: they also stand as a step of their own, one row per
            # "request" at its own position, for the last entry of the schedule.
            req = lay.req[lay.rows]
            ar = np.arange(R + 1, dtype=np.int32)
            kv_r = (lay.pos[lay.rows] + 1).astype(np.int32)
            ctx.tail = StepContext(
                num_tokens=R, num_requests=R, token_ids=self._to_device(lay.ids[lay.rows]),
                positions=self._to_device(lay.pos[lay.rows]), token_req=self._to_device(ar[:R]),
                cu_q=self._to_device(ar), kv_lens=self._to_device(kv_r),
                block_tables=[self._to_device(np.ascontiguousarray(t[req])) for t in host_tables] if R else tables,
                slots=[self._to_device(s[lay.rows]) for s in lay.slots],
                state_slots=self._to_device(lay.state_slots[req]),
                q_lens=[1] * R, kv_lens_host=kv_r.tolist(), max_q_len=1, max_kv_len=int(kv_r.max()) if R else 0,
                prior_positions_settled=False)
            ctx.tail_rows = rows
        return ctx, rows

    def build_context(self, entries: Sequence[StepEntry]):
        """Check, reserve pages and lay the batch out on the device (no graph)."""
        self._check(entries)
        self._reserve(entries)
        return self._context(self._layout(entries))

    def graph_width(self, rows: int) -> int:
        """The captured width that a decode batch of ``rows`` requests replays: itself up to 8
        rows, the next multiple of 8 beyond (fewer graphs to capture and keep while a batch
        drains); no padding when a mixer keeps fixed state, whose slots padding rows would share."""
        if rows <= 8 or self.cache.has_fixed_state:
            return rows
        return -(-rows // 8) * 8

    # ------------------------------------------------------------------ the step
    def _graphable(self, entries: Sequence[StepEntry], lay: _Layout) -> bool:
        return (self.use_graphs and all(n == 1 for n in lay.q_lens)
                and all(list(e.want) == [0] for e in entries)
                and int(lay.kv_lens.max()) <= self.graph_max_kv_len)

    def step(self, entries: Sequence[StepEntry], ids_device: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the batch; returns float32 logits ``[wanted, vocab]`` on the device, in the
        order of the entries and of their ``want`` lists.  (With graphs the tensor is a
        static buffer that the next decode step of the same size overwrites.)
        ``ids_device`` (int32, one id per token of the step) replaces the entries' token ids on
        the device: a step launched before the host has read the ids that the previous step
        chose; the entries then carry placeholders."""
        self._check(entries)
        self._reserve(entries)
        self.h2d_bytes = 0
        try:
            lay = self._layout(entries)
            if self._graphable(entries, lay):
                width = self.graph_width(lay.B)
                g = self._graphs.get(width)
                if g is None:
                    g = self._graphs[width] = _DecodeGraph(self, width)
                g.fill(lay, lay.serials)
                self.h2d_bytes += g.nbytes
                if ids_device is not None:
                    g.d["ids"][:lay.B].copy_(ids_device, non_blocking=True)
                logits = g.run(self)
            else:
                ctx, rows = self._context(lay)
                if ids_device is not None:
                    ctx.token_ids = ids_device
                    if ctx.tail is not None:
                        ctx.tail.token_ids = ops.gather_rows(ids_device, ctx.tail_rows)
                logits = self.model.forward(ctx, self.layer_caches, rows)
        except Exception:
            for e in entries:
                self.cache.rollback(e.request_id)
            for g in self._graphs.values():       # rolled-back pages may come back as others
                g.forget_rows()
            raise
        for e in entries:
            self.cache.commit(e.request_id)
        self.steps_run += 1
        return logits

    def status_words(self) -> List[torch.Tensor]:
        """The device words (int32[1]) that kernels of a step may set: bad input seen by the model's
        kernels, and a bounded wait that a tensor-core kernel gave up (its output is then unfinished)."""
        return [self.model.status, ops.tc_status(self.device)]

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input (an id outside the table, non-finite logits) or gave
        up a bounded wait.  Waits for the device."""
        codes = torch.cat(self.status_words()).tolist()
        if any(codes):
            for w in self.status_words():
                w.zero_()
            raise RuntimeError(ops.describe_status(max(codes)))
