"""The scheduler above the step function.  The reference has none: its batch is fixed by the caller,
every prompt runs whole in one step and finished requests stay in the batch
(tiny_llm/pipeline/pipeline.cpp:100-229).  Decisions here, in the order they are taken each step:

  1. Requests that are running and have one token to run (decoding) get that token.
  2. Running requests with more tokens to run (a prompt not yet finished, or a request that was
     pushed out and recomputes) get a portion of at most `chunk` tokens, oldest first, while the
     step's token budget lasts.
  3. Waiting requests are admitted first come, first served, while a state slot is free, budget
     is left and the pages of their first portion fit.
  4. When pages run out for a running request, the most recently admitted running request is
     pushed out: its pages and slot are given back and it returns to the head of the waiting queue
     with its prompt and everything it generated, to be recomputed.  A request that could never
     fit (prompt + max_new_tokens beyond the model's positions or the pool) is refused on arrival,
     so the oldest request always makes progress.
  5. A request ends on an end-of-sequence token, on max_new_tokens, or at the model's last
     position; its pages and slot are given back at once."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache import CacheManager
from ..sampling import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1   # stands in a request's generated tokens for an id that was sampled but not read back yet


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    generated: List[int] = field(default_factory=list)
    state: str = WAITING
    num_computed: int = 0          # tokens of prompt + generated that are in the cache
    finish_reason: Optional[str] = None
    times_pushed_out: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def remaining(self) -> int:
        return self.num_tokens - self.num_computed

    def token_slice(self, start: int, count: int) -> List[int]:
        """Tokens [start, start + count) of prompt + generated, without joining the two lists."""
        n = len(self.prompt)
        if start >= n:
            return self.generated[start - n: start - n + count]
        if start + count <= n:
            return self.prompt[start: start + count]
        return self.prompt[start:] + self.generated[: start + count - n]


@dataclass
class Scheduled:
    request: Request
    start: int        # first token of the portion, as an index into prompt + generated
    count: int
    samples: bool     # the portion ends at the request's last token: its logits are wanted


class RequestRefused(ValueError):
    pass


class Scheduler:
    def __init__(self, cache: CacheManager, max_positions: int, max_tokens_per_step: int = 2048,
                 max_requests_per_step: int = 64, chunk: int = 512, eos_token_ids: Sequence[int] = ()):
        self.cache = cache
        self.max_positions = max_positions
        self.max_tokens_per_step = max_tokens_per_step
        self.max_requests_per_step = max_requests_per_step
        self.chunk = chunk
        self.eos = set(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []   # in order of admission
        self.counters = {"steps": 0, "tokens": 0, "pushed_out": 0, "finished": 0}

    # ---- arrival
    def add(self, request: Request) -> None:
        n = len(request.prompt)
        if n == 0:
            raise RequestRefused(f"request {request.rid!r}: empty prompt")
        total = n + request.params.max_new_tokens
        if total > self.max_positions:
            raise RequestRefused(f"request {request.rid!r}: prompt of {n} tokens + max_new_tokens "
                                 f"{request.params.max_new_tokens} exceeds the model's {self.max_positions} positions")
        for g in self.cache.groups:
            # the fewest tokens the request must be able to hold pages for: all of them, or, in a group
            # with a window, the window and the token being written, rounded out to whole pages at both
            # ends (pages behind the window come back only after the step that passed them)
            most = total if g.need.window is None else min(total, g.need.window + 2 * g.page_size)
            if g.pages_for(most) > g.pool.num_pages:
                raise RequestRefused(f"request {request.rid!r}: {most} tokens need {g.pages_for(most)} pages, "
                                     f"the pool has {g.pool.num_pages}")
        request.state = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step's plan
    def _push_out(self, victim: Request) -> None:
        self.cache.free_request(victim.rid)
        self.running.remove(victim)
        victim.state = WAITING
        victim.num_computed = 0
        victim.times_pushed_out += 1
        self.waiting.appendleft(victim)
        self.counters["pushed_out"] += 1

    def schedule(self) -> List[Scheduled]:
        plan: List[Scheduled] = []
        budget = self.max_tokens_per_step
        decoding = [r for r in self.running if r.remaining == 1]
        filling = [r for r in self.running if r.remaining > 1]
        for req in decoding + filling:
            if req.state != RUNNING:
                continue  # pushed out while an earlier request was served
            if budget == 0 or len(plan) == self.max_requests_per_step:
                break
            n = min(req.remaining, self.chunk, budget)
            while not self.cache.reserve(req.rid, n):
                victim = self.running[-1]
                if victim is req and len(self.running) == 1:
                    # alone and still short: a smaller portion may fit
                    n = self._largest_portion_that_fits(req, n)
                    if n == 0:
                        raise RuntimeError(f"request {req.rid!r} cannot make progress although it runs alone")
                    continue
                plan = [s for s in plan if s.request is not victim]
                self._push_out(victim)
                if victim is req:
                    break
            if req.state != RUNNING:
                continue
            plan.append(Scheduled(req, req.num_computed, n, req.num_computed + n == req.num_tokens))
            budget -= n
        # admission
        while self.waiting and budget > 0 and len(plan) < self.max_requests_per_step:
            req = self.waiting[0]
            if self.cache.slots.num_free == 0:
                break
            n = min(req.remaining, self.chunk, budget)
            if self.cache.add_request(req.rid) is None:
                break
            if not self.cache.reserve(req.rid, n):
                if not self.running and not plan:
                    # nothing else holds pages: a smaller first portion fits (add() made sure of that)
                    n = self._largest_portion_that_fits(req, n)
                if n == 0 or not self.cache.reserve(req.rid, n):
                    self.cache.free_request(req.rid)
                    break
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            plan.append(Scheduled(req, req.num_computed, n, req.num_computed + n == req.num_tokens))
            budget -= n
        return plan

    def _largest_portion_that_fits(self, req: Request, n: int) -> int:
        while n > 0 and not self.cache.can_reserve(req.rid, n):
            n -= 1
        return n

    # ---- after the step
    def finish_step(self, plan: List[Scheduled], sampled: Dict[Hashable, int]) -> List[Request]:
        """`sampled[rid]` is the token drawn for every planned request whose portion sampled.  The
        cache was committed by the step function.  Returns the requests that ended."""
        ended = []
        self.counters["steps"] += 1
        for s in plan:
            req = s.request
            req.num_computed += s.count
            self.counters["tokens"] += s.count
            if not s.samples:
                continue
            tok = sampled[req.rid]
            req.generated.append(tok)
            reason = None
            if self.ends_sequence(req, tok):
                reason = "eos"
            elif len(req.generated) >= req.params.max_new_tokens:
                reason = "length"
            elif req.num_tokens >= self.max_positions:
                reason = "positions"
            if reason:
                self.finish(req, reason)
                ended.append(req)
        return ended

    def ends_sequence(self, req: Request, tok: int) -> bool:
        return tok in self.eos and not req.params.ignore_eos

    def finish(self, req: Request, reason: str) -> None:
        """The request has ended: its pages and slot go back at once."""
        req.state = FINISHED
        req.finish_reason = reason
        self.cache.free_request(req.rid)
        self.running.remove(req)
        self.counters["finished"] += 1
