"""SwiGLU feed-forward: m = (silu(y Wg^T) * (y Wu^T)) Wd^T, no biases
(tiny_llm/parser/llama_parser.cpp:225-249; tiny_llm/ops/cuda/silu.cu:7-12; arithmetic.cu:7-22).

The reference runs gate and up as two products over the same input, then SiLU, then the product.
Here the two weights are fused at load time into one matrix whose rows alternate in blocks of
`block` gate rows and `block` up rows, so that one output tile of the fused product holds matching
gate and up columns and SiLU * up can be taken in 32-bit where the accumulators are."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import COMPUTE, WeightSpec
from .registry import register_part


def interleave_gate_up(wg: torch.Tensor, wu: torch.Tensor, block: int) -> torch.Tensor:
    """Rows [2 g block, 2 g block + block) are gate rows [g block, (g+1) block); the next `block`
    rows are the matching up rows.  `block` must divide the number of rows."""
    i, h = wg.shape
    assert i % block == 0
    g = i // block
    return torch.stack([wg.view(g, block, h), wu.view(g, block, h)], dim=1).reshape(2 * i, h).contiguous()


def gate_up_block(intermediate_size: int) -> int:
    for b in (128, 64, 32, 16, 8, 4, 2):
        if intermediate_size % b == 0:
            return b
    return 1


class SwiGLU:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.block = gate_up_block(intermediate_size)
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self, prefix: str):
        i, h = self.intermediate_size, self.hidden_size
        return [WeightSpec(prefix + "gate_proj.weight", (i, h), COMPUTE),
                WeightSpec(prefix + "up_proj.weight", (i, h), COMPUTE),
                WeightSpec(prefix + "down_proj.weight", (h, i), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.w_gate_up = interleave_gate_up(weights[prefix + "gate_proj.weight"],
                                            weights[prefix + "up_proj.weight"], self.block)
        self.w_down = weights[prefix + "down_proj.weight"]

    def forward(self, ctx, h, resid) -> None:
        t = h.shape[0]
        act = ctx.workspace.get("ffn_act", (t, self.intermediate_size), ctx.dtype)
        ops.linear_swiglu(h, self.w_gate_up, act, self.block, ctx.workspace)
        ops.linear(act, self.w_down, resid, accumulate=True)


register_part("ffn", "swiglu", SwiGLU)
