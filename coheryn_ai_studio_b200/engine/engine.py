"""The engine a user talks to: requests in, tokens out.

``Engine.generate`` is the Python entry point; its options carry the reference's names
and meanings (crates/coheryn-engine/src/inference.rs:69-142 ``GenerationOptions`` /
``GenerationResult``; crates/coheryn-cli/src/main.rs:136-190): ``max_tokens`` (default
128), ``temperature`` / ``top_k`` / ``top_p`` / ``seed`` and the three penalties,
``stop_tokens``, ``context`` (admission capacity, at most the model's positions).
"""
from __future__ import annotations

import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..sampling.sampler import DeviceSampler, RequestSampler, SamplingParams
from .loading import load_model, parse_dtype
from .scheduler import FINISH_LENGTH, Request, RequestRefused, Scheduler
from .step import StepEntry, StepRunner


@dataclass
class GenerationResult:
    """Field names follow crates/coheryn-engine/src/inference.rs:117-142."""

    token_ids: List[int]
    prompt_tokens: int
    reused_prompt_tokens: int
    completion_tokens: int
    finish_reason: str
    prefill_ms: float
    decode_ms: float
    first_token_ms: Optional[float]
    text: str = ""
    preemptions: int = 0

    def to_dict(self) -> Dict:
        return asdict(self)


@dataclass
class _Timing:
    start: float
    first_token: Optional[float] = None
    end: Optional[float] = None


@dataclass
class _InFlight:
    """A step that has been launched and whose chosen ids have not been read yet."""
    plan: list
    sampling: List[Request]
    pending: object


class Engine:
    def __init__(self, model, *, dtype="bfloat16", context: int = 4096, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 2048, page_size: int = 16,
                 num_pages: Optional[int] = None, kv_cache_tokens: Optional[int] = None,
                 prefix_reuse: bool = True, eos_token_ids: Sequence[int] = (), use_graphs: bool = True,
                 lookahead: bool = True):
        """``model`` is a DecoderModel on the device.  The cache pool holds ``num_pages``
        pages per group, or enough for ``kv_cache_tokens`` tokens, or by default enough for
        ``max_num_seqs`` requests of ``context`` tokens.  ``use_graphs`` replays decode steps
        from CUDA graphs (one per batch size, captured at first use).  ``lookahead`` launches
        the next decode step before the host has read the ids the current one chose (they go
        from step to step on the device), so the GPU does not idle while the host keeps its
        books; the tokens a request receives are the same."""
        self.model = model
        spec = model.spec
        if context < 1 or context > spec.max_positions:
            raise ValueError(f"context {context} must be in 1..={spec.max_positions} "
                             "(the model's positions)")
        self.context = context
        if num_pages is None:
            tokens = kv_cache_tokens if kv_cache_tokens is not None else context * max_num_seqs
            num_pages = -(-tokens // page_size)
        self.cache = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule],
                                  parse_dtype(dtype), model.runtime.device, page_size=page_size,
                                  num_pages=num_pages, max_requests=max_num_seqs,
                                  prefix_reuse=prefix_reuse)
        self.runner = StepRunner(model, self.cache, use_graphs=use_graphs, graph_max_kv_len=context)
        self.scheduler = Scheduler(self.cache, context, max_num_seqs, max_num_batched_tokens)
        self.sampler = DeviceSampler(model.runtime.device)
        self.eos_token_ids = tuple(eos_token_ids)
        self._timing: Dict[str, _Timing] = {}
        self._requests: Dict[str, Request] = {}
        self._counter = 0
        self.lookahead = bool(lookahead)
        self._inflight: Optional[_InFlight] = None

    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0", **kwargs) -> "Engine":
        config, model = load_model(model_dir, dtype, device)
        kwargs.setdefault("eos_token_ids", getattr(config, "eos_token_ids", ()))
        return cls(model, dtype=dtype, **kwargs)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], max_tokens: int = 128,
                    params: Optional[SamplingParams] = None, stop_tokens: Sequence[int] = (),
                    request_id: Optional[str] = None) -> str:
        params = params or SamplingParams()
        params.validate(self.model.spec.vocab_size)
        if len(stop_tokens) > 16:
            raise RequestRefused("custom stop limits exceeded")     # main.rs:236-241
        V = self.model.spec.vocab_size
        for t in prompt:
            if not 0 <= int(t) < V:
                raise RequestRefused("token ID outside vocabulary")
        if request_id is None:
            request_id = f"req-{self._counter}"
            self._counter += 1
        if request_id in self._requests:
            raise RequestRefused(f"request id {request_id!r} is in use")
        req = Request(request_id, [int(t) for t in prompt], int(max_tokens), params,
                      tuple(int(t) for t in stop_tokens) + self.eos_token_ids)
        self.scheduler.add(req)
        self._requests[request_id] = req
        self._timing[request_id] = _Timing(time.perf_counter())
        if req.max_tokens == 0:
            self.scheduler.finish(req, FINISH_LENGTH)
            self._timing[request_id].end = time.perf_counter()
        return request_id

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one step
    def _launch(self, plan, ids_device=None) -> _InFlight:
        """Run a plan's batch and start the selection of its tokens; nothing waits."""
        entries = [StepEntry(s.request.request_id, s.tokens, [len(s.tokens) - 1] if s.samples else [])
                   for s in plan]
        if ids_device is not None:      # the entries' ids are placeholders until the previous step's are read
            for s in plan:
                self.cache.mark_unknown(s.request.request_id, self.cache.length(s.request.request_id))
        logits = self.runner.step(entries, ids_device=ids_device)
        self.scheduler.advance(plan)
        sampling = [s.request for s in plan if s.samples]
        pending = self.sampler.launch(logits, [r.sampler for r in sampling], extra_status=self.runner.status_words())
        return _InFlight(plan, sampling, pending)

    def step(self) -> List[tuple]:
        """Schedule, run, sample.  Returns (request_id, token, finished) for every token
        sampled in the step that this call completes."""
        cur, self._inflight = self._inflight, None
        if cur is None:
            plan = self.scheduler.schedule()
            if not plan:
                if self.scheduler.has_work():
                    raise RuntimeError("the scheduler found nothing to run although requests are pending")
                return []
            cur = self._launch(plan)
        # The step after this one, when it can be planned without this one's tokens: launched now,
        # fed on the device with the ids being chosen, it runs while the host keeps its books.
        if self.lookahead and cur.pending.ids is not None and len(cur.sampling) == len(cur.plan):
            ahead = self.scheduler.lookahead(cur.plan)
            if ahead is not None:
                self._inflight = self._launch(ahead, ids_device=cur.pending.ids)
        tokens = self.sampler.finish(cur.pending)
        now = time.perf_counter()
        events = []
        for req, tok in zip(cur.sampling, tokens):
            if req.finished:           # ended (or aborted) while this step was in flight: its token is dropped
                continue
            if self._inflight is not None:
                # the step launched ahead reserved this id's place with a placeholder
                self.cache.patch_token(req.request_id, req.num_tokens, tok)
            tm = self._timing[req.request_id]
            if tm.first_token is None:
                tm.first_token = now
            done = self.scheduler.append_token(req, tok)
            if done:
                tm.end = now
            events.append((req.request_id, tok, done))
        if not self.scheduler.has_work():
            self._inflight = None      # what was launched ahead has nobody left to serve
        return events

    # ------------------------------------------------------------------ results
    def result(self, request_id: str, forget: bool = True) -> GenerationResult:
        req, tm = self._requests[request_id], self._timing[request_id]
        end = tm.end if tm.end is not None else time.perf_counter()
        first = tm.first_token
        res = GenerationResult(
            token_ids=list(req.output), prompt_tokens=len(req.prompt),
            reused_prompt_tokens=req.reused_prompt_tokens, completion_tokens=len(req.output),
            finish_reason=req.finish_reason or "cancelled",
            prefill_ms=((first if first is not None else end) - tm.start) * 1e3,
            decode_ms=(end - first) * 1e3 if first is not None else 0.0,
            first_token_ms=(first - tm.start) * 1e3 if first is not None else None,
            preemptions=req.preemptions)
        if forget:
            del self._requests[request_id], self._timing[request_id]
        return res

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 128,
                 params=None, stop_tokens: Sequence[int] = (),
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Generate for a list of prompts (token ids) with continuous batching.  ``params``
        is one SamplingParams for all or a list; ``on_token(prompt_index, token)`` streams."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        ids = [self.add_request(p, max_tokens, pr, stop_tokens) for p, pr in zip(prompts, params)]
        index = {rid: i for i, rid in enumerate(ids)}
        while self.scheduler.has_work():
            for rid, tok, _ in self.step():
                if on_token is not None and rid in index:
                    on_token(index[rid], tok)
        return [self.result(rid) for rid in ids]
