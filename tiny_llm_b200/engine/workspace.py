"""Named scratch buffers of the step.  A buffer is as large as the largest request seen for its
name (or as `reserve` made it), so the addresses stay put once the engine is warm."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}    # (name, dtype, shape) -> the view handed out before
        self.frozen = False

    def reserve(self, name: str, numel: int, dtype: torch.dtype) -> None:
        key = (name, dtype)
        cur = self._buffers.get(key)
        if cur is None or cur.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow to {numel} elements "
                                   f"while its address is pinned by a captured graph")
            self._buffers[key] = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._drop_views(key)

    def _drop_views(self, key) -> None:
        for k in [k for k in self._views if k[0] == key[0] and k[1] == key[1]]:
            del self._views[k]

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        vkey = (name, dtype, tuple(shape))
        view = self._views.get(vkey)       # a step asks for the same few views over and over: making one costs 3 us
        if view is not None:
            return view
        numel = 1
        for s in shape:
            numel *= int(s)
        self.reserve(name, numel, dtype)
        view = self._buffers[(name, dtype)][:numel].view(*shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[vkey] = view
        return view

    def get_zeroed(self, name: str, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A buffer that holds zeros when it is handed out for the first time and that every user
        hands back zeroed (the consumer kernel clears what it reads): split-K sums accumulate there."""
        numel = 1
        for s in shape:
            numel *= int(s)
        key = (name, dtype)
        cur = self._buffers.get(key)
        if cur is None or cur.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while its address is pinned")
            self._buffers[key] = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            self._drop_views(key)
        return self._buffers[key][:numel].view(*shape)
