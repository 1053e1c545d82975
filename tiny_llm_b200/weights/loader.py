"""Weights by tensor name.  Every part declares the tensors it wants (`WeightSpec`); the loader
checks the whole set against the file before it touches the device and reports everything that
is wrong in ONE error.  The reference looks tensors up by the same checkpoint names one at a time
and stops at the first failure (tiny_llm/runtime/cuda/cuda_runtime.cpp:353-361,
tiny_llm/weight_managers/safetensors/weight_manager.cpp:87-93)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Mapping, Tuple, Union

import torch

from .errors import WeightError
from .safetensors_io import SafetensorsFile

# how a stored tensor is kept on the device
COMPUTE = "compute"      # matrices of matrix products: the engine's dtype (bfloat16 or float32)
FLOAT32 = "float32"      # small vectors that scale in 32-bit (norm weights): always float32
INT32 = "int32"          # integer tables
AS_STORED = "as_stored"  # a tensor that is stored in 32-bit stays 32-bit; 16-bit floats go to the engine's dtype


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    keep: str = COMPUTE


def _convert(t: torch.Tensor, spec: WeightSpec, dtype: torch.dtype) -> torch.Tensor:
    if spec.keep == INT32:
        return t.to(torch.int32)
    if spec.keep == FLOAT32:
        return t.to(torch.float32)
    if spec.keep == AS_STORED and t.dtype in (torch.float32, torch.int32):
        return t
    return t.to(dtype)


class _DictSource:
    def __init__(self, d: Mapping[str, torch.Tensor]):
        self.d = d

    def keys(self):
        return self.d.keys()

    def __contains__(self, k):
        return k in self.d

    def shape(self, k):
        return tuple(self.d[k].shape)

    def dtype(self, k):
        return self.d[k].dtype

    def get(self, k):
        return self.d[k]

    def close(self):
        pass


def open_source(source: Union[str, Mapping[str, torch.Tensor]]):
    """A model folder (its model.safetensors), a .safetensors file, or a dict of tensors."""
    if isinstance(source, (str, os.PathLike)):
        path = os.fspath(source)
        if os.path.isdir(path):
            path = os.path.join(path, "model.safetensors")
        return SafetensorsFile(path)
    return _DictSource(source)


def check_against(specs: Mapping[str, WeightSpec], src) -> None:
    missing = sorted(n for n in specs if n not in src)
    unexpected = sorted(n for n in src.keys() if n not in specs)
    wrong = []
    for n, s in specs.items():
        if n not in src:
            continue
        if tuple(src.shape(n)) != tuple(s.shape):
            wrong.append(f"{n}: expected shape {list(s.shape)}, found {list(src.shape(n))}")
        elif s.keep == INT32 and src.dtype(n).is_floating_point:
            wrong.append(f"{n}: expected an integer table, found {src.dtype(n)}")
        elif s.keep != INT32 and not src.dtype(n).is_floating_point:
            wrong.append(f"{n}: expected floating point, found {src.dtype(n)}")
    if missing or unexpected or wrong:
        lines = ["weights do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or kind ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightError("\n".join(lines))


def load_state(specs: Mapping[str, WeightSpec], source, dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Checks the whole set, then converts and moves tensor by tensor."""
    src = open_source(source)
    try:
        check_against(specs, src)
        out = {}
        for n, s in specs.items():
            out[n] = _convert(src.get(n), s, dtype).to(device).contiguous()
        return out
    finally:
        src.close()
