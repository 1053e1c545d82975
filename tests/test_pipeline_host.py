"""The generation loop's chaining of decode steps, on the host (no GPU): the step function and the
sampler are replaced by bookkeeping, the scheduler and the cache manager are the real ones.

While requests only decode, `Pipeline.step` launches step N + 1 before it has read the ids that
step N sampled.  Whatever a request ran after an end-of-sequence id has to be dropped, also when the
step that ran too far ended the request by length or at the model's last position."""
import pytest

from tiny_llm_b200.cache import CacheManager, KVNeed
from tiny_llm_b200.engine.pipeline import Pipeline
from tiny_llm_b200.engine.scheduler import Scheduler
from tiny_llm_b200.sampling import SamplingParams

EOS = 99


class FakeRunner:
    """Commits the cache as the step function does and counts what it was given."""

    def __init__(self, cache):
        self.cache = cache
        self.steps = []

    def step(self, entries, device_tokens=None):
        for e in entries:
            assert self.cache.reserve(e.rid, len(e.tokens))
        for e in entries:
            self.cache.commit(e.rid, len(e.tokens))
        self.steps.append(([(e.rid, list(e.tokens)) for e in entries], device_tokens is not None))
        return [e.rid for e in entries if e.want]     # stands for the logits: who is sampled


class FakeSampler:
    """Hands out scripted ids per request: script[rid][n] is the n-th id the request draws."""

    def __init__(self, script):
        self.script = script
        self.collected = 0

    def launch(self, logits, params, counters):
        class Ticket:
            device_out = object()
        t = Ticket()
        t.ids = [self.script[rid][n] for rid, n in zip(logits, counters)]
        return t

    def collect(self, ticket):
        self.collected += 1
        return ticket.ids


def make(script, max_pos=64, max_tokens=256):
    cache = CacheManager([KVNeed(1, 16)], max_tokens=max_tokens, page_size=4, max_slots=4)
    sched = Scheduler(cache, max_pos, max_tokens_per_step=32, max_requests_per_step=4, chunk=16, eos_token_ids=(EOS,))
    runner = FakeRunner(cache)
    return Pipeline.from_parts(runner, sched, FakeSampler(script)), runner, cache


def generate(pipe, prompts, max_new, **kw):
    reqs = []
    for rid, p in prompts.items():
        pipe.add_request(p, SamplingParams(max_new_tokens=max_new, do_sample=False, **kw), rid=rid)
        reqs.append(pipe.scheduler.waiting[-1])
    steps = 0
    while pipe.has_work():
        pipe.step()
        steps += 1
        assert steps < 200
    pipe._forget(pipe._resolve_pending())
    return {r.rid: (r.generated, r.finish_reason) for r in reqs}


@pytest.mark.parametrize("eos_at", range(0, 8))
def test_end_of_sequence_cuts_the_result_wherever_it_falls(eos_at):
    """max_new_tokens 8: an end-of-sequence id at every place, the last two included (where the
    chained step that ran too far ends the request by length before the id is read)."""
    ids = [10 + i for i in range(8)]
    ids[eos_at] = EOS
    pipe, runner, cache = make({"a": ids})
    out = generate(pipe, {"a": [1, 2, 3]}, 8)
    assert out["a"] == (ids[: eos_at + 1], "eos")
    assert cache.groups[0].pool.num_used == 0 and cache.slots.num_free == 4
    free, _, _ = make({"a": ids})
    assert generate(free, {"a": [1, 2, 3]}, 8, ignore_eos=True)["a"] == (ids, "length")


def test_decode_steps_are_chained_and_results_do_not_depend_on_it():
    script = {"a": [10, 11, 12, 13, EOS, 15, 16, 17], "b": [20, 21, 22, 23, 24, 25, EOS, 27], "c": [30] * 8}
    pipe, runner, cache = make(script)
    out = generate(pipe, {"a": [1, 2, 3], "b": [4, 5], "c": [6]}, 8)
    assert out == {"a": ([10, 11, 12, 13, EOS], "eos"), "b": ([20, 21, 22, 23, 24, 25, EOS], "eos"), "c": ([30] * 8, "length")}
    assert pipe.counters["chained"] > 0
    assert any(chained for _, chained in runner.steps)
    assert cache.groups[0].pool.num_used == 0 and cache.slots.num_free == 4


def test_the_last_position_of_the_model_ends_a_request_and_an_earlier_eos_still_wins():
    ids = [10, 11, 12, EOS, 14, 15]
    pipe, _, cache = make({"a": ids}, max_pos=8)
    # prompt of 3 + 5 new = the model's 8 positions: "positions" would end it after the fifth id
    assert generate(pipe, {"a": [1, 2, 3]}, 5)["a"] == ([10, 11, 12, EOS], "eos")
    pipe, _, cache = make({"a": [10, 11, 12, 13, EOS, 15]}, max_pos=8)
    assert generate(pipe, {"a": [1, 2, 3]}, 5)["a"] == ([10, 11, 12, 13, EOS], "eos")
    assert cache.groups[0].pool.num_used == 0


def test_a_request_that_can_never_be_admitted_raises_instead_of_spinning():
    pipe, _, cache = make({"a": [1] * 8})
    pipe.add_request([1, 2, 3], SamplingParams(max_new_tokens=4, do_sample=False), rid="a")
    while cache.slots.num_free:                      # somebody else holds every slot
        cache.slots.acquire(("held", cache.slots.num_free))
    with pytest.raises(RuntimeError, match="cannot be admitted"):
        pipe.step()
