"""The scheduler's decisions (no GPU): the step function is replaced by bookkeeping."""
import random

import pytest

from tiny_llm_b200.cache import CacheManager, KVNeed
from tiny_llm_b200.engine.scheduler import FINISHED, Request, RequestRefused, Scheduler
from tiny_llm_b200.sampling import SamplingParams


def make(max_tokens=64, page=4, slots=4, budget=16, chunk=8, max_pos=64, eos=()):
    cache = CacheManager([KVNeed(1, 16)], max_tokens=max_tokens, page_size=page, max_slots=slots)
    return Scheduler(cache, max_pos, max_tokens_per_step=budget, max_requests_per_step=slots, chunk=chunk,
                     eos_token_ids=eos), cache


def run_step(s, cache, token=9):
    """What the engine does with a plan: run (commit) and sample `token` for every finished portion."""
    plan = s.schedule()
    for p in plan:
        cache.commit(p.request.rid, p.count)
    sampled = {p.request.rid: (token(p.request) if callable(token) else token) for p in plan if p.samples}
    return plan, s.finish_step(plan, sampled)


def req(rid, n, new=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_new_tokens=new, do_sample=False, **kw))


def test_prompts_are_cut_into_portions_under_the_budget_and_decodes_go_first():
    s, cache = make(budget=16, chunk=8)
    s.add(req("a", 20))
    s.add(req("b", 3))
    plan, _ = run_step(s, cache)
    assert [(p.request.rid, p.start, p.count, p.samples) for p in plan] == [("a", 0, 8, False), ("b", 0, 3, True)]
    plan, _ = run_step(s, cache)   # b decodes first, then a's next portion
    assert [(p.request.rid, p.start, p.count, p.samples) for p in plan] == [("b", 3, 1, True), ("a", 8, 8, False)]
    plan, _ = run_step(s, cache)
    assert [(p.request.rid, p.count, p.samples) for p in plan] == [("b", 1, True), ("a", 4, True)]
    assert sum(p.count for p in plan) <= 16


def test_budget_limits_admission():
    s, cache = make(budget=10, chunk=8)
    for i in range(3):
        s.add(req(i, 8))
    plan, _ = run_step(s, cache)
    assert [(p.request.rid, p.count) for p in plan] == [(0, 8), (1, 2)]
    plan, _ = run_step(s, cache)
    assert [(p.request.rid, p.count) for p in plan] == [(0, 1), (1, 6), (2, 3)]


def test_finishes_on_eos_length_and_positions_and_frees_at_once():
    s, cache = make(eos=(7,), max_pos=12)
    s.add(req("len", 3, new=2))
    s.add(req("eos", 3, new=5))
    s.add(req("ign", 3, new=3, ignore_eos=True))
    s.add(req("pos", 8, new=4))
    tok = lambda r: 7 if r.rid in ("eos", "ign") else 9
    ended = []
    while s.has_work():
        _, e = run_step(s, cache, tok)
        ended += e
        cache.check()
    reasons = {r.rid: (r.finish_reason, len(r.generated)) for r in ended}
    assert reasons == {"len": ("length", 2), "eos": ("eos", 1), "ign": ("length", 3), "pos": ("length", 4)}
    assert cache.groups[0].pool.num_used == 0 and cache.slots.num_free == 4
    assert all(r.state == FINISHED for r in ended)
    s2, cache2 = make(max_pos=10)
    s2.add(req("p", 8, new=2))
    out = []
    while s2.has_work():
        out += run_step(s2, cache2)[1]
    assert out[0].finish_reason in ("length", "positions") and out[0].num_tokens == 10


def test_requests_that_can_never_fit_are_refused():
    s, _ = make(max_tokens=16, max_pos=64)
    with pytest.raises(RequestRefused, match="pages"):
        s.add(req("big", 20, new=4))
    with pytest.raises(RequestRefused, match="positions"):
        s.add(req("long", 62, new=4))
    with pytest.raises(RequestRefused, match="empty"):
        s.add(Request("none", [], SamplingParams()))


def test_when_pages_run_out_the_newest_request_is_pushed_out_and_recomputed():
    # 6 pages of 4 tokens; two requests of 8 + up to 8 new tokens cannot both stay
    s, cache = make(max_tokens=24, page=4, budget=32, chunk=16, max_pos=64)
    s.add(req("old", 8, new=8))
    s.add(req("new", 8, new=8))
    pushed = False
    steps = 0
    ended = []
    while s.has_work():
        plan, e = run_step(s, cache)
        ended += e
        cache.check()
        steps += 1
        assert steps < 100
        if s.counters["pushed_out"] and not pushed:
            pushed = True
            victim = s.waiting[0]
            assert victim.rid == "new" and victim.num_computed == 0 and victim.generated  # keeps what it generated
            assert not cache.has_request("new")
    assert pushed and {r.rid for r in ended} == {"old", "new"}
    assert all(len(r.generated) == 8 for r in ended)
    assert ended[0].rid == "old"                      # the oldest request always makes progress
    assert cache.groups[0].pool.num_used == 0


@pytest.mark.parametrize("seed", range(5))
def test_random_load_always_drains(seed):
    rng = random.Random(seed)
    s, cache = make(max_tokens=48, page=4, slots=3, budget=12, chunk=5, max_pos=40, eos=(3,))
    todo = [req(i, rng.randint(1, 20), new=rng.randint(1, 12)) for i in range(12)]
    done = []
    steps = 0
    while todo or s.has_work():
        if todo and rng.random() < 0.5:
            s.add(todo.pop())
        plan, e = run_step(s, cache, lambda r: rng.randint(0, 9))
        assert sum(p.count for p in plan) <= 12 and len(plan) <= 3
        assert len({p.request.rid for p in plan}) == len(plan)
        done += e
        cache.check()
        steps += 1
        assert steps < 2000
    assert len(done) == 12 and cache.groups[0].pool.num_used == 0 and cache.slots.num_free == 3


def test_a_windowed_group_admits_by_its_window_and_shrinks_the_first_portion():
    """A pool that holds a window and a little more: a long prompt is admitted with a first portion
    that fits, runs to its end with pages coming back behind the window, and a request whose window
    can never fit is refused on arrival instead of waiting for ever."""
    cache = CacheManager([KVNeed(1, 16, window=8)], max_tokens=20, page_size=4, max_slots=2)
    s = Scheduler(cache, 64, max_tokens_per_step=32, max_requests_per_step=2, chunk=32)
    s.add(req("w", 40, new=3))
    steps = 0
    while s.has_work():
        plan, _ = run_step(s, cache)
        assert plan, "the scheduler planned nothing although a request waits and nothing runs"
        cache.check()
        steps += 1
        assert steps < 100
    assert cache.groups[0].pool.num_used == 0
    small = CacheManager([KVNeed(1, 16, window=16)], max_tokens=8, page_size=4, max_slots=2)
    with pytest.raises(RequestRefused):
        Scheduler(small, 64, chunk=8).add(req("x", 30))
