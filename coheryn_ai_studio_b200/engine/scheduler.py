"""Continuous batching: admit requests, cut prompts into portions under a token budget,
decode, finish and free.

What the reference's scheduler does per token with one-token lanes, a width of at most 16
and capacity reserved up front (crates/coheryn-api/src/scheduler.rs:321-415,
crates/coheryn-api/src/scheduler/batching.rs:163-219) is done here per step with pages
allocated on demand:

* every step gives each running request one token if it is decoding, else the next
  portion of its prompt, oldest request first, until ``max_num_batched_tokens`` is spent;
  a portion may be any size down to one token;
* waiting requests are admitted first-in first-out while fewer than ``max_num_seqs`` run
  and the budget and the free pages allow their first portion;
* a request is refused at submission only when it can never run: an empty prompt,
  ``prompt + max_tokens`` beyond the context (crates/coheryn-engine/src/inference/
  generation.rs:152-161), or more pages than the whole pool has;
* when pages run out in the middle of generation, idle cached pages are evicted first
  (the pool does that by itself), then nothing new is admitted, then the most recently
  admitted running request is preempted: its pages are freed and it goes back to the head
  of the waiting queue with its prompt and the tokens generated so far, to be computed
  again later.  Sampling state is kept, so its output is the same as without preemption.

The decisions are taken by the native planner (``csrc/host_engine.cpp``: ``Planner``), which
works on the cache manager's native book; :class:`Scheduler` is its Python face and keeps the
user-facing :class:`Request` records (token lists, sampler state, results) in step with it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..cache.pages import host
from ..sampling.sampler import RequestSampler, SamplingParams

FINISH_STOP, FINISH_LENGTH, FINISH_CANCELLED = "stop", "length", "cancelled"
PLACEHOLDER_TOKEN = 0     # stands for an id that is still on the device (see Scheduler.lookahead)


class RequestRefused(ValueError):
    """The request can never run on this engine."""


@dataclass(eq=False)     # a request is itself: lists of requests compare by identity
class Request:
    request_id: str
    prompt: List[int]
    max_tokens: int
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: Tuple[int, ...] = ()
    output: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens whose keys/values are in the cache
    reused_prompt_tokens: int = 0
    finish_reason: Optional[str] = None
    preemptions: int = 0
    sampler: Optional[RequestSampler] = None
    arrival: int = 0
    handle: int = -1                 # the native planner's number for this request

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_slice(self, start: int, stop: int) -> List[int]:
        """tokens[start:stop] without building the whole list."""
        n = len(self.prompt)
        if stop <= n:
            return self.prompt[start:stop]
        if start >= n:
            return self.output[start - n:stop - n]
        return self.prompt[start:] + self.output[:stop - n]

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class Scheduled:
    request: Request
    tokens: List[int]
    samples: bool        # the step's last token of this request yields a sampled token


_REASONS = {1: FINISH_STOP, 2: FINISH_LENGTH, 3: FINISH_CANCELLED}
_REASON_CODES = {v: k for k, v in _REASONS.items()}


def _ints(values):
    n = len(values)
    return (ctypes.c_int * max(n, 1))(*[int(v) for v in values]), n


class Scheduler:
    def __init__(self, cache: CacheManager, context: int, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 2048):
        if max_num_seqs < 1 or max_num_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        self.cache, self.context = cache, context
        self.max_num_batched_tokens = max_num_batched_tokens
        self._lib = host()
        self._h = self._lib.coheryn_planner_new(cache.book_handle, int(context), int(max_num_seqs),
                                                int(max_num_batched_tokens))
        if not self._h:
            raise RuntimeError("the native planner could not be made")
        self.max_num_seqs = int(self._lib.coheryn_planner_max_seqs(self._h))
        self._jobs: List[Request] = []          # by handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.coheryn_planner_delete(h)

    # ------------------------------------------------------------------ views
    def _list(self, which: int) -> List[Request]:
        cap = max(len(self._jobs), 1)
        out = (ctypes.c_int * cap)()
        n = self._lib.coheryn_planner_list(self._h, which, out, cap)
        return [self._jobs[out[i]] for i in range(n)]

    @property
    def running(self) -> List[Request]:
        """The running requests in order of admission (a copy)."""
        return self._list(2)

    @property
    def waiting(self) -> List[Request]:
        """The waiting requests in queue order (a copy)."""
        return self._list(3)

    @property
    def stats(self) -> dict:
        out = (ctypes.c_longlong * 6)()
        self._lib.coheryn_planner_stats(self._h, out)
        return {"steps": out[0], "preemptions": out[1], "admitted": out[2], "finished": out[3],
                "scheduled_tokens": out[4], "max_batch_width": out[5]}

    # ------------------------------------------------------------------ submission
    def _refuse(self, code: int, req: Request) -> None:
        ps = self.cache.page_size
        need = -(-(len(req.prompt) + max(req.max_tokens - 1, 0)) // ps)
        raise RequestRefused({
            20: "the prompt holds no token",
            21: "max_tokens must not be negative",
            22: f"prompt ({len(req.prompt)}) + max_tokens ({req.max_tokens}) exceeds the context of {self.context}",
            23: f"the request needs {need} cache pages; the pool has {self.cache.num_pages}",
            25: f"request id {req.request_id!r} is in use",
        }.get(code, f"the planner refused the request (status {code})"))

    def add(self, req: Request) -> None:
        prompt, n = _ints(req.prompt)
        stops, n_stops = _ints(req.stop_token_ids)
        handle = ctypes.c_int(-1)
        code = self._lib.coheryn_planner_add(self._h, str(req.request_id).encode(), prompt, n, int(req.max_tokens), stops,
                                             n_stops, 1 if req.params.penalised else 0, ctypes.byref(handle))
        if code:
            self._refuse(code, req)
        self._register(req, handle.value)
        if req.sampler is None:
            req.sampler = RequestSampler(req.params, req.prompt)

    def _register(self, req: Request, handle: int) -> None:
        req.handle = handle
        req.arrival = handle
        assert handle == len(self._jobs)
        self._jobs.append(req)

    def adopt_running(self, req: Request, computed: int) -> None:
        """Take in a request whose pages are already in the cache (``computed`` tokens of its prompt
        committed under its id): it counts as running from now on.  For callers that fill the cache
        by other means than running the prompt."""
        prompt, n = _ints(req.prompt)
        handle = ctypes.c_int(-1)
        code = self._lib.coheryn_planner_adopt(self._h, str(req.request_id).encode(), prompt, n, int(req.max_tokens),
                                               int(computed), ctypes.byref(handle))
        if code:
            self._refuse(code, req)
        self._register(req, handle.value)
        req.num_computed = computed
        if req.sampler is None:
            req.sampler = RequestSampler(req.params, req.prompt)

    def has_work(self) -> bool:
        return bool(self._lib.coheryn_planner_has_work(self._h))

    # ------------------------------------------------------------------ one step's plan
    def _plan(self, n: int, placeholder: bool = False) -> List[Scheduled]:
        cap = max(n, 1)
        jobs, starts, counts, samples = ((ctypes.c_int * cap)() for _ in range(4))
        self._lib.coheryn_planner_plan(self._h, jobs, starts, counts, samples, cap)
        out = []
        for i in range(n):
            req = self._jobs[jobs[i]]
            toks = [PLACEHOLDER_TOKEN] * counts[i] if placeholder else req.token_slice(starts[i], starts[i] + counts[i])
            out.append(Scheduled(req, toks, bool(samples[i])))
        return out

    def schedule(self) -> List[Scheduled]:
        n = self._lib.coheryn_planner_schedule(self._h)
        cap = max(len(self._jobs), 1)
        buf = (ctypes.c_int * cap)()
        for i in range(self._lib.coheryn_planner_list(self._h, 0, buf, cap)):      # preempted in this step
            req = self._jobs[buf[i]]
            req.num_computed = 0
            req.preemptions += 1
        for i in range(self._lib.coheryn_planner_list(self._h, 1, buf, cap)):      # admitted in this step
            req = self._jobs[buf[i]]
            req.num_computed = int(self._lib.coheryn_planner_job(self._h, req.handle, 0))
            req.reused_prompt_tokens = int(self._lib.coheryn_planner_job(self._h, req.handle, 1))
            self.cache.zero_state(req.request_id)
        return self._plan(n)

    def lookahead(self, plan: Sequence[Scheduled]) -> Optional[List[Scheduled]]:
        """The plan of the step AFTER ``plan`` when that can be said before ``plan``'s tokens
        are known: ``plan`` decodes every running request, nobody waits, none of the requests can
        end by length or context with the token ``plan`` yields, and the pages are there.  The
        entries carry a placeholder id (the real one is still on the device).  Call after
        ``advance(plan)``.  None when the ordinary ``schedule`` has to decide."""
        if not plan:
            return None
        jobs, n = _ints([s.request.handle for s in plan])
        counts, _ = _ints([len(s.tokens) for s in plan])
        samples, _ = _ints([1 if s.samples else 0 for s in plan])
        if not self._lib.coheryn_planner_lookahead(self._h, n, jobs, counts, samples):
            return None
        return self._plan(n, placeholder=True)

    # ------------------------------------------------------------------ after the step
    def advance(self, plan: Sequence[Scheduled]) -> None:
        jobs, n = _ints([s.request.handle for s in plan])
        counts, _ = _ints([len(s.tokens) for s in plan])
        self._lib.coheryn_planner_advance(self._h, n, jobs, counts)
        for s in plan:
            s.request.num_computed += len(s.tokens)

    def append_token(self, req: Request, token: int) -> bool:
        """Record a sampled token; returns True when the request is finished.  The last
        sampled token is not run through the model (generation.rs:386-388)."""
        req.output.append(token)
        reason = self._lib.coheryn_planner_append_token(self._h, req.handle, int(token))
        if reason > 0:
            req.finish_reason = _REASONS[reason]
        return req.finished

    def finish(self, req: Request, reason: str) -> None:
        req.finish_reason = reason
        self._lib.coheryn_planner_finish(self._h, req.handle, _REASON_CODES.get(reason, 3))

    def abort(self, request_id: str) -> bool:
        for req in self.running + self.waiting:
            if req.request_id == request_id:
                self.finish(req, FINISH_CANCELLED)
                return True
        return False
