"""The Python entry point, in the manner of the reference's Pipeline
(tiny_llm/pipeline/pipeline.hpp:12-41): built from a model folder, `apply(prompts, max_new_tokens,
do_sample, temperature, top_k, top_p)` returns the generated sequences.  Prompts and results are
token ids (the tokenizer is outside the engine).  Underneath run the scheduler, the step function
and the device-side sampler; requests may also be added one by one and stepped."""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..sampling import Sampler, SamplingParams
from .loading import load_model, make_runner, parse_dtype
from .scheduler import PENDING, RUNNING, Request, Scheduled, Scheduler
from .step import StepEntry


class _Pending:
    """The ids a step sampled that the host has not read yet: where they go in each request."""

    def __init__(self, ticket, requests: List[Request], index: List[int]):
        self.ticket, self.requests, self.index = ticket, requests, index
        self.rids = [r.rid for r in requests]


class Pipeline:
    def __init__(self, model_path: str, dtype="bfloat16", device: int = 0, page_size: int = 16,
                 max_tokens: Optional[int] = None, max_requests: int = 64, max_tokens_per_step: int = 2048,
                 chunk: Optional[int] = None):
        """`max_tokens`: tokens the cache pool holds (default: max_requests x the model's positions,
        capped at 1M tokens).  `chunk`: the largest portion of one prompt in one step (default: the step's whole
        token budget; measured at the TinyLlama sizes a step of 512 prompt tokens runs at 233,000 tokens a second and a
        step of 2,048 at 448,000, so a prompt is cut no finer than the budget asks)."""
        if not chunk:
            chunk = max_tokens_per_step
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the engine runs on a B200 and has no other path")
        self.device = torch.device(f"cuda:{device}" if isinstance(device, int) else device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        if isinstance(model_path, tuple):   # (config, loaded model): see from_model
            self.config, self.model = model_path
        else:
            self.config, self.model = load_model(model_path, self.dtype, self.device)
        spec = self.model.spec
        if max_tokens is None:
            max_tokens = min(max_requests * spec.max_positions, 1 << 20)
        self.runner = make_runner(self.model, self.dtype, self.device, max_tokens=max_tokens, page_size=page_size,
                                  max_requests=max_requests, max_tokens_per_step=max_tokens_per_step)
        self.scheduler = Scheduler(self.runner.cache, spec.max_positions, max_tokens_per_step=max_tokens_per_step,
                                   max_requests_per_step=max_requests, chunk=chunk,
                                   eos_token_ids=spec.eos_token_ids)
        self.sampler = Sampler(self.device, spec.vocab_size, max_rows=max(2, max_requests + max_requests % 2))
        self._ids = itertools.count()
        self.requests: Dict[Hashable, Request] = {}
        self._pending: Optional[_Pending] = None
        self.counters = {"steps": 0, "chained": 0}

    @classmethod
    def from_model(cls, config, model, **kwargs) -> "Pipeline":
        """A pipeline around a model that is already loaded on the device (kwargs as the constructor's)."""
        return cls((config, model), **kwargs)

    @classmethod
    def from_parts(cls, runner, scheduler: Scheduler, sampler) -> "Pipeline":
        """A pipeline around a given step function, scheduler and sampler (anything with `step`,
        `cache`; `launch`, `collect`): what the host-side tests of the chaining logic use."""
        self = object.__new__(cls)
        self.runner, self.scheduler, self.sampler = runner, scheduler, sampler
        self._ids = itertools.count()
        self.requests = {}
        self._pending = None
        self.counters = {"steps": 0, "chained": 0}
        return self

    # ---- request by request
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, rid: Hashable = None):
        rid = next(self._ids) if rid is None else rid
        req = Request(rid, list(prompt), params or SamplingParams())
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def step(self) -> List[Request]:
        """Plans one step, runs it, samples, and returns the requests that ended.

        While requests only decode, steps are chained: the ids a step samples stay on the device and
        feed the next step directly, and the host reads them one step late, while the next step already
        runs.  A request that turns out to have sampled an end-of-sequence token has then run one step
        too many; that step's result is dropped.  Everything else (arrivals, portions of prompts,
        requests ending by length, pages running short) is resolved before the next plan is made."""
        ended: List[Request] = []
        if self._pending is not None and not self._can_chain():
            ended += self._resolve_pending()
        plan = self.scheduler.schedule()
        if not plan:
            if self._pending is not None:
                ended += self._resolve_pending()
            elif not ended and not self.scheduler.running and self.scheduler.waiting:
                # nothing runs, nothing was read back, and still the oldest waiting request was not
                # admitted: the next call would find the same, so say so instead of spinning
                req = self.scheduler.waiting[0]
                raise RuntimeError(f"request {req.rid!r} cannot be admitted although nothing else is running "
                                   f"(free slots {self.runner.cache.slots.num_free}, free pages "
                                   f"{[g.pool.num_free for g in self.runner.cache.groups]})")
            return self._forget(ended)
        entries = []
        sampling: List[Scheduled] = []
        for s in plan:
            toks = s.request.token_slice(s.start, s.count)
            if self._pending is not None:
                toks = [0]   # the real id is still on the device
            entries.append(StepEntry(s.request.rid, toks, [s.count - 1] if s.samples else []))
            if s.samples:
                sampling.append(s)
        device_tokens = None
        if self._pending is not None:
            if [s.request.rid for s in plan] != self._pending.rids or any(s.count != 1 for s in plan):
                raise RuntimeError("a chained step was planned for other requests than the step before it")
            device_tokens = self._pending.ticket.device_out
        logits = self.runner.step(entries, device_tokens=device_tokens)
        self.counters["steps"] += 1
        self.counters["chained"] += device_tokens is not None
        ticket = None
        if sampling:
            ticket = self.sampler.launch(logits, [s.request.params for s in sampling],
                                         [len(s.request.generated) for s in sampling])
        previous = self._pending
        finished = self.scheduler.finish_step(plan, {s.request.rid: PENDING for s in sampling})
        self._pending = None
        if ticket is not None:
            self._pending = _Pending(ticket, [s.request for s in sampling],
                                     [len(s.request.generated) - 1 for s in sampling])
        if previous is not None:
            ended += self._apply(previous)          # the ids of the step before: copied long ago
        if finished:                                 # ended by length: their last id is needed now
            ended += self._resolve_pending()
            ended += [r for r in finished if r not in ended]
        return self._forget(ended)

    def _forget(self, ended: List[Request]) -> List[Request]:
        for r in ended:
            self.requests.pop(r.rid, None)
        return ended

    def _can_chain(self) -> bool:
        """True when the next plan is certain to be: the very requests that sampled last step, one
        token each, nothing admitted, nothing pushed out."""
        sched, pend = self.scheduler, self._pending
        if sched.waiting or [r.rid for r in sched.running] != pend.rids:
            return False
        if any(r.remaining != 1 for r in sched.running):
            return False
        cache = self.runner.cache
        need = [0] * len(cache.groups)
        for r in sched.running:
            for gi, m in enumerate(cache.pages_missing(r.rid, 1)):
                need[gi] += m
        return all(n <= g.pool.num_free for n, g in zip(need, cache.groups))

    def _apply(self, pending: "_Pending") -> List[Request]:
        """Writes a step's sampled ids where their placeholders stand; a request whose id is an
        end-of-sequence token ends there (whatever it ran after that is dropped)."""
        ended = []
        for req, idx, tok in zip(pending.requests, pending.index, self.sampler.collect(pending.ticket)):
            if idx >= len(req.generated):
                continue   # the request ended before this id was sampled: a step too many
            req.generated[idx] = tok
            if self.scheduler.ends_sequence(req, tok):
                # whatever the request ran after this id is dropped, also when the chained step that
                # followed has already ended it by length or at the model's last position
                del req.generated[idx + 1:]
                if req.state == RUNNING:
                    self.scheduler.finish(req, "eos")
                    ended.append(req)
                else:
                    req.finish_reason = "eos"
        return ended

    def _resolve_pending(self) -> List[Request]:
        pending, self._pending = self._pending, None
        return self._apply(pending) if pending is not None else []

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ---- the reference's call
    def apply(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256, do_sample: bool = True,
              temperature: float = 0.7, top_k: int = 50, top_p: float = 0.95, seed: int = 0,
              ignore_eos: bool = False) -> List[List[int]]:
        """Generates for every prompt; request i draws from the random stream seed + i."""
        reqs = []
        for i, p in enumerate(prompts):
            params = SamplingParams(max_new_tokens=max_new_tokens, do_sample=do_sample, temperature=temperature,
                                    top_k=top_k, top_p=top_p, seed=seed + i, ignore_eos=ignore_eos)
            rid = self.add_request(p, params)
            reqs.append(self.scheduler.waiting[-1])
            assert reqs[-1].rid == rid
        while self.has_work():
            self.step()
        self._forget(self._resolve_pending())
        return [r.generated for r in reqs]

    generate = apply
