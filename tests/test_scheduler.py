"""The scheduler's decisions on the host: admission, portions under the token budget,
decoding, finishing and freeing, and what happens when pages run out."""
import pytest
import torch

from coheryn_ai_studio_b200.cache import CacheManager
from coheryn_ai_studio_b200.engine.scheduler import Request, RequestRefused, Scheduler
from coheryn_ai_studio_b200.parts import PagedKV


def make(pages=16, page=4, context=64, seqs=4, budget=8, prefix=False):
    cache = CacheManager([PagedKV(1, 4, None)], [None], torch.float32, torch.device("cpu"),
                         page_size=page, num_pages=pages, max_requests=8, prefix_reuse=prefix)
    return cache, Scheduler(cache, context, seqs, budget)


def run_step(cache, sched, next_token=lambda req: 1000 + len(req.output)):
    """What the engine does around the model: reserve, commit, sample."""
    plan = sched.schedule()
    for s in plan:
        assert cache.reserve(s.request.request_id, s.tokens), "the plan did not fit the pool"
    for s in plan:
        cache.commit(s.request.request_id)
    sched.advance(plan)
    for s in plan:
        if s.samples:
            sched.append_token(s.request, next_token(s.request))
    cache.check()
    return plan


def test_refusals():
    cache, sched = make(pages=4, page=4, context=32)
    with pytest.raises(RequestRefused, match="no token"):
        sched.add(Request("a", [], 4))
    with pytest.raises(RequestRefused, match="context"):
        sched.add(Request("a", [1] * 30, 3))
    with pytest.raises(RequestRefused, match="pages"):
        sched.add(Request("a", [1] * 17, 2))       # 18 tokens in cache = 5 pages > 4
    sched.add(Request("a", [1] * 16, 1))           # the last sampled token is never cached


def test_prompt_is_cut_under_the_budget_then_decodes():
    cache, sched = make(budget=8)
    r = Request("a", list(range(19)), 3)
    sched.add(r)
    sizes = []
    while sched.has_work():
        plan = run_step(cache, sched)
        sizes.append([len(s.tokens) for s in plan])
    assert sizes == [[8], [8], [3], [1], [1]]
    assert r.output == [1000, 1001, 1002] and r.finish_reason == "length"
    assert cache.available_pages() == [16] and not cache.requests


def test_decodes_go_first_and_share_the_step_with_a_prompt():
    cache, sched = make(budget=8)
    a, b = Request("a", [1, 2, 3], 5), Request("b", list(range(20)), 2)
    sched.add(a)
    run_step(cache, sched)                          # a: whole prompt, first token
    sched.add(b)
    plan = run_step(cache, sched)
    assert [(s.request.request_id, len(s.tokens), s.samples) for s in plan] == [("a", 1, True), ("b", 7, False)]
    plan = run_step(cache, sched)
    assert [(s.request.request_id, len(s.tokens)) for s in plan] == [("a", 1), ("b", 7)]
    plan = run_step(cache, sched)
    assert [(s.request.request_id, len(s.tokens), s.samples) for s in plan] == [("a", 1, True), ("b", 6, True)]


def test_first_in_first_out_and_width_limit():
    cache, sched = make(seqs=2, budget=100)
    reqs = [Request(f"r{i}", [1] * 5, 2) for i in range(4)]
    for r in reqs:
        sched.add(r)
    assert [s.request.request_id for s in run_step(cache, sched)] == ["r0", "r1"]
    assert [s.request.request_id for s in run_step(cache, sched)] == ["r0", "r1"]   # both finish here
    assert [s.request.request_id for s in run_step(cache, sched)] == ["r2", "r3"]
    assert sched.stats["max_batch_width"] == 2


def test_stop_token_finishes_and_stays_in_the_ids():
    cache, sched = make()
    r = Request("a", [1, 2], 10, stop_token_ids=(1001,))
    sched.add(r)
    while sched.has_work():
        run_step(cache, sched)
    assert r.output == [1000, 1001] and r.finish_reason == "stop"


def test_newcomer_waits_for_room():
    cache, sched = make(pages=6, page=4, budget=100)     # 24 tokens of cache
    a, b = Request("a", [1] * 14, 4), Request("b", [2] * 12, 2)
    sched.add(a); sched.add(b)
    plan = run_step(cache, sched)
    assert [s.request.request_id for s in plan] == ["a"]          # b's 12 tokens need 3 pages, 2 are free
    assert sched.stats["preemptions"] == 0 and len(sched.waiting) == 1
    while not a.finished:
        run_step(cache, sched)
    while sched.has_work():
        run_step(cache, sched)
    assert b.output == [1000, 1001]


def test_preemption_recomputes_and_keeps_the_output():
    def outputs(pages):
        cache, sched = make(pages=pages, page=4, context=64, budget=100)
        reqs = [Request("a", [1] * 7, 12), Request("b", [2] * 7, 12), Request("c", [3] * 6, 12)]
        for r in reqs:
            sched.add(r)
        steps = 0
        while sched.has_work():
            run_step(cache, sched, next_token=lambda req: hash((req.request_id, len(req.output))) % 500)
            steps += 1
            assert steps < 500
        assert cache.available_pages() == [pages]
        return [r.output for r in reqs], sched.stats["preemptions"], [r.preemptions for r in reqs]
    roomy, p0, _ = outputs(pages=32)
    tight, p1, per_request = outputs(pages=8)             # 32 tokens for three requests that grow to 18
    assert p0 == 0 and p1 > 0
    assert tight == roomy
    assert per_request[0] == 0, "the oldest request is never the victim"


def test_abort_frees_pages():
    cache, sched = make()
    a = Request("a", [1] * 9, 5)
    sched.add(a)
    run_step(cache, sched)
    assert sched.abort("a") and a.finish_reason == "cancelled"
    assert cache.available_pages() == [16] and not sched.has_work()
    assert not sched.abort("a")


def test_prefix_reuse_shortens_the_prompt_work():
    cache, sched = make(pages=16, page=4, budget=100, prefix=True)
    prompt = list(range(50, 63))
    a = Request("a", prompt, 1)
    sched.add(a)
    run_step(cache, sched)
    b = Request("b", prompt, 1)
    sched.add(b)
    plan = run_step(cache, sched)
    assert len(plan[0].tokens) == 1 and b.reused_prompt_tokens == 12


def test_a_request_whose_pages_are_already_there_is_adopted():
    """``adopt_running``: the caller filled the cache under the request's id; the planner takes the
    request in as running and decodes it from where the cache ends."""
    cache, sched = make(pages=8, page=4)
    prompt = list(range(1, 10))
    assert cache.admit("x") is not None and cache.reserve("x", prompt[:-1])
    cache.commit("x")
    r = Request("x", prompt, 3)
    sched.adopt_running(r, len(prompt) - 1)
    assert sched.running == [r] and not sched.waiting and r.num_computed == 8
    plan = sched.schedule()
    assert len(plan) == 1 and plan[0].tokens == [9] and plan[0].samples
    with pytest.raises(RequestRefused):
        sched.adopt_running(Request("x", prompt, 3), 8)                  # the id is in use


def test_the_planner_forgets_the_tokens_of_finished_requests():
    cache, sched = make(pages=16, page=4)
    reqs = [Request(f"r{i}", [1 + i] * 5, 2) for i in range(3)]
    for r in reqs:
        sched.add(r)
    while sched.has_work():
        run_step(cache, sched)
    assert all(r.finish_reason == "length" and len(r.output) == 2 for r in reqs)
    assert sched.stats["finished"] == 3 and cache.available_pages() == [16] and not cache.requests
    for r in reqs:        # the native side keeps the numbers of a finished job, not its token lists
        assert sched._lib.coheryn_planner_job(sched._h, r.handle, 4) == 0
        assert sched._lib.coheryn_planner_job(sched._h, r.handle, 3) == 2
