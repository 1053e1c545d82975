"""Sampling options, with the names, defaults and meanings of the reference's command line
(main.cpp:10-18) and of Pipeline::apply (tiny_llm/pipeline/pipeline.cpp:100-103, 156-164)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 256   # cap on generated tokens
    do_sample: bool = True      # False: greedy (first maximum)
    temperature: float = 0.7    # logits are divided by it
    top_k: int = 50             # keep the k largest logits; 0 keeps all
    top_p: float = 0.95         # drop the least likely tokens while their mass stays <= 1 - p
    seed: int = 0               # the request's random stream; draws do not depend on the batch
    ignore_eos: bool = False    # keep generating past an end-of-sequence token

    def __post_init__(self):
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if self.do_sample and not self.temperature > 0:
            raise ValueError("temperature must be positive when sampling")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must lie in [0, 1]")
