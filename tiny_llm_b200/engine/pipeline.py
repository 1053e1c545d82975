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
from .scheduler import Request, Scheduled, Scheduler
from .step import StepEntry


class Pipeline:
    def __init__(self, model_path: str, dtype="bfloat16", device: int = 0, page_size: int = 16,
                 max_tokens: Optional[int] = None, max_requests: int = 64, max_tokens_per_step: int = 2048,
                 chunk: int = 512):
        """`max_tokens`: tokens the cache pool holds (default: max_requests x the model's positions,
        capped at 1M tokens)."""
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

    @classmethod
    def from_model(cls, config, model, **kwargs) -> "Pipeline":
        """A pipeline around a model that is already loaded on the device (kwargs as the constructor's)."""
        return cls((config, model), **kwargs)

    # ---- request by request
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, rid: Hashable = None):
        rid = next(self._ids) if rid is None else rid
        req = Request(rid, list(prompt), params or SamplingParams())
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def step(self) -> List[Request]:
        """Plans one step, runs it, samples, and returns the requests that ended in it."""
        plan = self.scheduler.schedule()
        if not plan:
            return []
        entries = []
        sampling: List[Scheduled] = []
        for s in plan:
            toks = s.request.token_slice(s.start, s.count)
            entries.append(StepEntry(s.request.rid, toks, [s.count - 1] if s.samples else []))
            if s.samples:
                sampling.append(s)
        logits = self.runner.step(entries)
        sampled = {}
        if sampling:
            toks = self.sampler.sample(logits, [s.request.params for s in sampling],
                                       [len(s.request.generated) for s in sampling])
            sampled = {s.request.rid: t for s, t in zip(sampling, toks)}
        ended = self.scheduler.finish_step(plan, sampled)
        for r in ended:
            self.requests.pop(r.rid, None)
        return ended

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
        return [r.generated for r in reqs]

    generate = apply
