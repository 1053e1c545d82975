"""From a model folder to a loaded model and its runner."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheManager
from ..config import load_config
from ..parts import DecoderModel
from ..weights import load_state
from .step import ModelRunner

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {name}")
        return name
    if name not in DTYPES:
        raise ValueError(f"unknown dtype {name!r}; choose bfloat16 or float32")
    return DTYPES[name]


def load_model(model_dir: str, dtype, device="cuda:0"):
    """Reads config.json, picks the model by its architecture name, loads the weights by name."""
    dtype = parse_dtype(dtype)
    config = load_config(model_dir)
    model = DecoderModel(config.model_spec())
    model.load(load_state(model.weight_specs(), model_dir, dtype, device, ignore=model.spec.ignored_weights))
    return config, model


def make_runner(model: DecoderModel, dtype, device="cuda:0", max_tokens: int = 8192, page_size: int = 16,
                max_requests: int = 64, max_tokens_per_step: Optional[int] = None) -> ModelRunner:
    """`max_tokens` sizes every cache group's pool (rounded up to whole pages)."""
    dtype = parse_dtype(dtype)
    cache = CacheManager(model.cache_needs(), max_tokens=max_tokens, page_size=page_size, max_slots=max_requests)
    cache.allocate_storage(dtype, device)
    return ModelRunner(model, cache, dtype, device,
                       max_tokens_per_step=max_tokens_per_step or min(max_tokens, 8192),
                       max_requests_per_step=max_requests)
