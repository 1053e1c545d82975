"""RMSNorm: y_j = (w_j x_j) / sqrt(mean_j(x_j^2) + eps), statistics in 32-bit
(tiny_llm/ops/cuda/norm.cu:16-49).  Any width; the reference stops at 2048."""
from __future__ import annotations

from .. import ops
from ..weights import FLOAT32, WeightSpec
from .registry import register_part


class RMSNorm:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = float(eps)
        self.weight = None

    def weight_specs(self, prefix: str):
        return [WeightSpec(prefix + ".weight", (self.size,), FLOAT32)]

    def load(self, prefix: str, weights) -> None:
        self.weight = weights[prefix + ".weight"]

    def forward(self, ctx, x, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.workspace.get("norm_out", (n, self.size), ctx.dtype)
        ops.rms_norm(x, self.weight, self.eps, out, rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
