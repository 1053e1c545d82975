"""Weights by tensor name.  Every part declares the tensors it wants (`WeightSpec`); the loader
checks the whole set against the file before it touches the device and reports everything that
is wrong in ONE error.  The reference looks tensors up by the same checkpoint names one at a time
and stops at the first failure (tiny_llm/runtime/cuda/cuda_runtime.cpp:353-361,
tiny_llm/weight_managers/safetensors/weight_manager.cpp:87-93)."""
from __future__ import annotations

import fnmatch
import json
import os
from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Sequence, Tuple, Union

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
    """`alias_of`: the tensor to stand in when `name` is not stored (an output matrix that a
    checkpoint leaves out because it equals the embedding table); both names then share one tensor."""
    name: str
    shape: Tuple[int, ...]
    keep: str = COMPUTE
    alias_of: Optional[str] = None


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


INDEX_NAME = "model.safetensors.index.json"


class ShardedSafetensors:
    """A checkpoint cut into several safetensors files with an index {"weight_map": {tensor name: file}}
    beside them (the layout large checkpoints are published in; the reference reads one file only,
    tiny_llm/pipeline/pipeline.cpp:67-68).  Shards are opened when a tensor of theirs is first asked for."""

    def __init__(self, folder: str):
        self.folder = folder
        path = os.path.join(folder, INDEX_NAME)
        try:
            with open(path) as f:
                index = json.load(f)
            self._file_of: Dict[str, str] = dict(index["weight_map"])
        except (OSError, ValueError, KeyError, TypeError) as e:
            raise WeightError(f"{path}: not a readable shard index ({e})") from None
        self._shards: Dict[str, SafetensorsFile] = {}
        for name, fname in self._file_of.items():    # every shard is opened once here: the check needs all shapes
            shard = self._shard(fname)
            if name not in shard:
                raise WeightError(f"{path}: tensor {name!r} is not in {fname} as the index says")

    def _shard(self, fname: str) -> SafetensorsFile:
        if fname not in self._shards:
            if os.path.basename(fname) != fname:
                raise WeightError(f"{self.folder}: the shard index names a file outside the folder: {fname!r}")
            self._shards[fname] = SafetensorsFile(os.path.join(self.folder, fname))
        return self._shards[fname]

    def keys(self):
        return self._file_of.keys()

    def __contains__(self, k):
        return k in self._file_of

    def shape(self, k):
        return self._shard(self._file_of[k]).shape(k)

    def dtype(self, k):
        return self._shard(self._file_of[k]).dtype(k)

    def get(self, k):
        return self._shard(self._file_of[k]).get(k)

    def close(self):
        for s in self._shards.values():
            s.close()


def open_source(source: Union[str, Mapping[str, torch.Tensor]]):
    """A model folder (its model.safetensors, or its shards by model.safetensors.index.json), a
    .safetensors file, or a dict of tensors."""
    if isinstance(source, (str, os.PathLike)):
        path = os.fspath(source)
        if os.path.isdir(path):
            single = os.path.join(path, "model.safetensors")
            if not os.path.isfile(single) and os.path.isfile(os.path.join(path, INDEX_NAME)):
                return ShardedSafetensors(path)
            path = single
        return SafetensorsFile(path)
    return _DictSource(source)


def check_against(specs: Mapping[str, WeightSpec], src, ignore: Sequence[str] = ()) -> None:
    """`ignore`: name patterns (fnmatch) of stored tensors that the model has no use for and that are
    known to be harmless; every other tensor the model does not want is an error."""
    missing = sorted(n for n, s in specs.items() if n not in src and not (s.alias_of and s.alias_of in src))
    unexpected = sorted(n for n in src.keys() if n not in specs and not any(fnmatch.fnmatchcase(n, p) for p in ignore))
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


def load_state(specs: Mapping[str, WeightSpec], source, dtype: torch.dtype, device,
               ignore: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Checks the whole set, then converts and moves tensor by tensor.  A tensor that is not stored
    but has an `alias_of` that is shares that tensor (no second copy on the device)."""
    src = open_source(source)
    try:
        check_against(specs, src, ignore)
        out = {}
        for n, s in specs.items():
            if n in src:
                out[n] = _convert(src.get(n), s, dtype).to(device).contiguous()
        for n, s in specs.items():
            if n not in out:
                other = specs.get(s.alias_of)
                if other is None or tuple(other.shape) != tuple(s.shape) or other.keep != s.keep:
                    raise WeightError(f"{n} is not stored and its stand-in {s.alias_of} has another shape or kind")
                out[n] = out[s.alias_of]
        return out
    finally:
        src.close()
