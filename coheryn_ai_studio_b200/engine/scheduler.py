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
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
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


class Scheduler:
    def __init__(self, cache: CacheManager, context: int, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 2048):
        if max_num_seqs < 1 or max_num_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        self.cache, self.context = cache, context
        self.max_num_seqs = min(max_num_seqs, cache.max_requests)
        self.max_num_batched_tokens = max_num_batched_tokens
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0
        self.stats = {"steps": 0, "preemptions": 0, "admitted": 0, "finished": 0,
                      "scheduled_tokens": 0, "max_batch_width": 0}

    # ------------------------------------------------------------------ submission
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise RequestRefused("the prompt holds no token")
        if req.max_tokens < 0:
            raise RequestRefused("max_tokens must not be negative")
        if len(req.prompt) + req.max_tokens > self.context:
            raise RequestRefused(f"prompt ({len(req.prompt)}) + max_tokens ({req.max_tokens}) "
                                 f"exceeds the context of {self.context}")
        need = -(-(len(req.prompt) + max(req.max_tokens - 1, 0)) // self.cache.page_size)
        if self.cache.groups and need > self.cache.num_pages:
            raise RequestRefused(f"the request needs {need} cache pages; the pool has "
                                 f"{self.cache.num_pages}")
        req.arrival = self._arrivals
        self._arrivals += 1
        if req.sampler is None:
            req.sampler = RequestSampler(req.params, req.prompt)
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step's plan
    def _preempt(self, victim: Request) -> None:
        """Free a running request's pages and put it back at the head of the queue."""
        self.running.remove(victim)
        self.cache.free(victim.request_id)
        victim.num_computed = 0
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)

    def _largest_fit(self, req: Request, n: int, reserved: List[int]) -> int:
        """The most tokens (at most n) of ``req`` that the free pages can take."""
        ps = self.cache.page_size
        for gi, avail in enumerate(self.cache.available_pages()):
            blocks = len(self.cache.block_table(req.request_id, gi)) + avail - reserved[gi]
            n = min(n, blocks * ps - self.cache.length(req.request_id))
        return max(n, 0)

    def schedule(self) -> List[Scheduled]:
        budget = self.max_num_batched_tokens
        plan: List[Scheduled] = []
        reserved = [0] * len(self.cache.groups)      # pages promised to earlier entries of this step
        preemptions_before = self.stats["preemptions"]

        def fits(req: Request, n: int) -> bool:
            need = self.cache.pages_needed(req.request_id, n)
            if not any(need):
                return True
            avail = self.cache.available_pages()
            return all(r + x <= a for r, x, a in zip(reserved, need, avail))

        def take(req: Request, n: int) -> None:
            for i, x in enumerate(self.cache.pages_needed(req.request_id, n)):
                reserved[i] += x
            toks = req.token_slice(req.num_computed, req.num_computed + n)
            plan.append(Scheduled(req, toks, req.num_computed + n == req.num_tokens))

        # running requests, oldest first
        preempted_ids = set()
        for req in sorted(self.running, key=lambda r: r.arrival):
            if budget == 0 or req.request_id in preempted_ids:      # nothing left, or preempted below
                continue
            n = min(req.num_tokens - req.num_computed, budget)
            while not fits(req, n):
                planned = {s.request.request_id for s in plan}
                victims = [r for r in self.running if r is not req and r.request_id not in planned]
                if not victims:
                    # Nobody left to preempt: run the part of the portion that fits.
                    n = self._largest_fit(req, n, reserved)
                    break
                victim = max(victims, key=lambda r: r.arrival)
                preempted_ids.add(victim.request_id)
                self._preempt(victim)
            if n == 0:
                continue
            take(req, n)
            budget -= n

        # admissions, first in first out; stop at the first that does not fit; none in a
        # step that had to preempt (the pool is short)
        preempted = self.stats["preemptions"] != preemptions_before
        while not preempted and self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            reused = self.cache.admit(req.request_id, req.tokens)
            if reused is None:
                break
            req.num_computed = reused
            n = min(req.num_tokens - req.num_computed, budget)
            if not fits(req, n):
                # Beside running requests a newcomer waits for room for its whole first
                # portion; alone it starts with what fits.
                n = 0 if (self.running or plan) else self._largest_fit(req, n, reserved)
            if n == 0:
                self.cache.free(req.request_id)
                req.num_computed = 0
                break
            if req.preemptions == 0:
                req.reused_prompt_tokens = reused
            self.waiting.popleft()
            self.running.append(req)
            self.stats["admitted"] += 1
            take(req, n)
            budget -= n

        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += sum(len(s.tokens) for s in plan)
        self.stats["max_batch_width"] = max(self.stats["max_batch_width"], len(plan))
        return plan

    def lookahead(self, plan: Sequence[Scheduled]) -> Optional[List[Scheduled]]:
        """The plan of the step AFTER ``plan`` when that can be said before ``plan``'s tokens
        are known: ``plan`` decodes every running request, nobody waits, none of the requests can
        end by length or context with the token ``plan`` yields, and the pages are there.  The
        entries carry a placeholder id (the real one is still on the device).  Call after
        ``advance(plan)``.  None when the ordinary ``schedule`` has to decide."""
        if self.waiting or not plan or len(plan) != len(self.running) or len(plan) > self.max_num_batched_tokens:
            return None
        reserved = [0] * len(self.cache.groups)
        avail = self.cache.available_pages()
        out: List[Scheduled] = []
        for s in plan:
            req = s.request
            if req.finished or not s.samples or len(s.tokens) != 1 or req not in self.running:
                return None
            if len(req.output) + 2 > req.max_tokens or req.num_tokens + 2 > self.context:
                return None
            if req.sampler is None or req.sampler.params.penalised:
                return None     # the penalties of the next step need this step's id
            for i, x in enumerate(self.cache.pages_needed(req.request_id, 1)):
                reserved[i] += x
            out.append(Scheduled(req, [PLACEHOLDER_TOKEN], True))
        if any(r > a for r, a in zip(reserved, avail)):
            return None
        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += len(out)
        self.stats["max_batch_width"] = max(self.stats["max_batch_width"], len(out))
        return out

    # ------------------------------------------------------------------ after the step
    def advance(self, plan: Sequence[Scheduled]) -> None:
        for s in plan:
            s.request.num_computed += len(s.tokens)

    def append_token(self, req: Request, token: int) -> bool:
        """Record a sampled token; returns True when the request is finished.  The last
        sampled token is not run through the model (generation.rs:386-388)."""
        req.output.append(token)
        if token in req.stop_token_ids:
            req.finish_reason = FINISH_STOP        # the stop token stays in the ids
        elif len(req.output) >= req.max_tokens:
            req.finish_reason = FINISH_LENGTH
        if req.finished:
            self.finish(req, req.finish_reason)
        return req.finished

    def finish(self, req: Request, reason: str) -> None:
        req.finish_reason = reason
        if req in self.running:
            self.running.remove(req)
            self.cache.free(req.request_id)
            self.stats["finished"] += 1
        elif req in self.waiting:
            self.waiting.remove(req)
            self.stats["finished"] += 1

    def abort(self, request_id: str) -> bool:
        for req in list(self.running) + list(self.waiting):
            if req.request_id == request_id:
                self.finish(req, FINISH_CANCELLED)
                return True
        return False
