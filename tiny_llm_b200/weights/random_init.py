"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a
seed.  Matrices are N(0, initializer_range), vectors that scale (norm weights) are 1.  Each tensor
has a generator of its own, keyed by the seed and the tensor's name, so a tensor's values do not
depend on which other tensors the model has.  The reference has no such mode; its tests fill
weights with ramps (tests/runtime/cuda/test_attention_runtime.cpp:165-174)."""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping

import torch

from .loader import COMPUTE, FLOAT32, INT32, WeightSpec
from .safetensors_io import save_safetensors


def _generator(seed: int, name: str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_state(specs: Mapping[str, WeightSpec], seed: int, std: float, dtype: torch.dtype,
                 device="cpu") -> Dict[str, torch.Tensor]:
    """Tensors for every spec.  On the CPU (the default, what `write_random_model` stores) the values
    are a function of (seed, name) alone; with a CUDA `device` they are drawn there from that
    device's generator, which is faster for large models but a different stream."""
    out = {}
    device = torch.device(device)
    for name, s in specs.items():
        if s.keep == INT32:
            out[name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
        elif s.keep == FLOAT32 and len(s.shape) == 1:
            out[name] = torch.ones(s.shape, dtype=dtype, device=device)
        else:
            g = _generator(seed, name)
            if device.type != "cpu":
                dg = torch.Generator(device=device)
                dg.manual_seed(g.initial_seed())
                g = dg
            t = torch.empty(s.shape, dtype=torch.float32, device=device)
            t.normal_(0.0, std, generator=g)
            out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.float32) -> str:
    """Writes `model_dir/config.json` and `model_dir/model.safetensors` for `config` (any registered
    configuration object) with weights drawn from `seed`, stored in `dtype`."""
    from ..parts.model import DecoderModel  # parts declare the tensors; imported late to keep weights/ free of parts/

    os.makedirs(model_dir, exist_ok=True)
    spec = config.model_spec()
    specs = DecoderModel(spec).weight_specs()
    state = random_state(specs, seed, spec.initializer_range, dtype)
    d = config.to_dict()
    d["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    save_safetensors(os.path.join(model_dir, "model.safetensors"), state,
                     metadata={"format": "pt", "seed": seed})
    return model_dir
