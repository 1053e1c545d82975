"""Reader and writer for the safetensors container: 8 bytes little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the raw little-endian tensor data.

The reference reads the same container through a Rust crate and accepts 32-bit floats only
(tiny_llm/weight_managers/safetensors/weight_manager.cpp:16-22, 52-116; src/lib.rs:24-147); this
reader takes every dtype the engine can convert."""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

from .errors import WeightError

# safetensors dtype code -> (numpy dtype that carries the bytes, torch dtype of the result)
_DTYPES = {
    "F64": (np.float64, torch.float64), "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16), "BF16": (np.int16, torch.bfloat16),
    "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32), "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8), "U8": (np.uint8, torch.uint8), "BOOL": (np.bool_, torch.bool),
}
_CODES = {v[1]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """A safetensors file mapped read-only; `get(name)` returns a CPU tensor that views the map."""

    def __init__(self, path: str):
        if not os.path.isfile(path):
            raise WeightError(f"no such weights file: {path}")
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise WeightError(f"{path}: header length {n} exceeds the file size")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            code, shape = e["dtype"], tuple(int(s) for s in e["shape"])
            begin, end = e["data_offsets"]
            if code not in _DTYPES:
                raise WeightError(f"{path}: tensor {name!r} has unsupported dtype {code}")
            want = int(np.prod(shape, dtype=np.int64)) * np.dtype(_DTYPES[code][0]).itemsize
            if end - begin != want or self._data_start + end > size:
                raise WeightError(f"{path}: tensor {name!r} has data offsets {begin}:{end} that do not "
                                  f"match shape {list(shape)} of {code}")
            self._entries[name] = (code, shape, begin, end)

    def keys(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name][0]][1]

    def get(self, name: str) -> torch.Tensor:
        code, shape, begin, end = self._entries[name]
        np_dtype, torch_dtype = _DTYPES[code]
        count = int(np.prod(shape, dtype=np.int64))
        arr = np.frombuffer(self._map, dtype=np_dtype, count=count, offset=self._data_start + begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; tensors from it are only read
            t = torch.from_numpy(arr.reshape(shape) if shape else arr.reshape(()))
        if torch_dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t

    def close(self):
        # tensors returned by get() view the map; callers copy (convert or move) before closing
        try:
            self._map.close()
        except BufferError:
            pass
        self._f.close()


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None) -> None:
    """Writes tensors in name order, each 8-byte aligned inside the data section."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _CODES:
            raise WeightError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.view(torch.int16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _CODES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hdr = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hdr += b" " * ((8 - len(hdr) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)))
        f.write(hdr)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
