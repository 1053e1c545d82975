"""Rotary position encoding, rotate-half pairing (i, i + rot_dim/2).  The angle table
ang[p, i] = p * theta^(-i / (rot_dim/2)) is made in 64-bit on the host and kept as 32-bit cos and
sin, as the reference's table kernel does (tiny_llm/ops/cuda/rope.cu:12-24); the rotation itself
runs in 32-bit inside the rotate-and-cache kernel (rope.cu:26-95 are its counterparts)."""
from __future__ import annotations

import torch

from .registry import register_part


class Rotary:
    fused = True  # the attention mixer may hand cos/sin to the fused rotate-and-cache kernel

    def __init__(self, head_dim: int, theta: float, max_positions: int, rot_dim=None):
        self.head_dim = head_dim
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rotary size {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        self.max_positions = max_positions
        self.cos = None
        self.sin = None

    def prepare(self, device) -> None:
        if self.cos is not None and self.cos.device == torch.device(device):
            return
        half = self.rot_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        p = torch.arange(self.max_positions, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -i / half)
        ang = p[:, None] * inv[None, :]
        self.cos = torch.cos(ang).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(ang).to(torch.float32).to(device).contiguous()


class NoPosition:
    """No position encoding: queries and keys go to the cache as they are."""
    fused = True
    cos = None
    sin = None
    rot_dim = 0

    def __init__(self, **_):
        pass

    def prepare(self, device) -> None:
        pass


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
