"""Named scratch buffers of the step.  A buffer is as large as the largest request seen for its
name (or as `reserve` made it), so the addresses stay put once the engine is warm."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.frozen = False

    def reserve(self, name: str, numel: int, dtype: torch.dtype) -> None:
        key = (name, dtype)
        cur = self._buffers.get(key)
        if cur is None or cur.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow to {numel} elements "
                                   f"while its address is pinned by a captured graph")
            self._buffers[key] = torch.empty(max(numel, 1), dtype=dtype, device=self.device)

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        self.reserve(name, numel, dtype)
        return self._buffers[(name, dtype)][:numel].view(*shape)

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
        return self._buffers[key][:numel].view(*shape)
