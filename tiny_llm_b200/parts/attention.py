"""Grouped-query attention over the paged cache.

One call: fused Q/K/V projection -> rotate Q and K and write K, V into the request's pages ->
attention of the step's queries over the cache -> output projection added into the residual
stream.  The reference runs this as seven launches with three separate projections
(tiny_llm/runtime/cuda/cuda_kernels.cpp:336-385); query head h reads key/value head
h // (heads / kv_heads) and scores are scaled by 1/sqrt(head_dim)
(tiny_llm/ops/cuda/flash_attention.cu:374-395).  A key at position j is visible to a query at
position p iff j <= p, and j > p - window when the part has a window."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache import KVNeed
from ..config.spec import PartSpec
from ..weights import COMPUTE, WeightSpec
from .registry import build_part, register_part


class GQAttention:

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window: Optional[int] = None, shares_cache: bool = False,
                 scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads evenly")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.window = window
        self.shares_cache = shares_cache
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.position = build_part("position", position)
        # launches this package's kernels only (a step through this part can be captured in a CUDA graph or run again
        # from a tape of its launches), unless the position encoding computes by itself
        self.graph_safe = bool(getattr(self.position, "fused", False) or getattr(self.position, "graph_safe", False))
        self.q_dim = num_heads * head_dim
        self.kv_dim = num_kv_heads * head_dim
        # a call that reads another call's cache projects queries only
        self.qkv_dim = self.q_dim if shares_cache else self.q_dim + 2 * self.kv_dim
        self.w_qkv = None
        self.w_o = None

    def cache_need(self):
        return None if self.shares_cache else KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def weight_specs(self, prefix: str):
        specs = [WeightSpec(prefix + "q_proj.weight", (self.q_dim, self.hidden_size), COMPUTE)]
        if not self.shares_cache:
            specs += [WeightSpec(prefix + "k_proj.weight", (self.kv_dim, self.hidden_size), COMPUTE),
                      WeightSpec(prefix + "v_proj.weight", (self.kv_dim, self.hidden_size), COMPUTE)]
        specs.append(WeightSpec(prefix + "o_proj.weight", (self.hidden_size, self.q_dim), COMPUTE))
        return specs

    def load(self, prefix: str, weights) -> None:
        names = ["q_proj.weight"] if self.shares_cache else ["q_proj.weight", "k_proj.weight", "v_proj.weight"]
        self.w_qkv = torch.cat([weights[prefix + n] for n in names], dim=0).contiguous()
        self.w_o = weights[prefix + "o_proj.weight"]
        self.position.prepare(self.w_o.device)

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        qkv = ctx.workspace.get("qkv", (t, self.qkv_dim), ctx.dtype)
        pos = self.position
        fused = getattr(pos, "fused", False)
        kv_slots = None if self.shares_cache else cache.slot_mapping
        if fused and ops.fused_qkv_preferred(t, self.qkv_dim, h.shape[1]) and ops.linear_rope_kv(
                h, self.w_qkv, qkv, ctx.batch.positions, pos.cos, pos.sin, self.num_heads, self.num_kv_heads,
                self.head_dim, cache.k, cache.v, kv_slots):
            pass    # projection, rotation and cache write were one kernel
        else:
            acc = None
            if fused and ops.prefers_split(h, self.w_qkv):
                # few rows: K is split over the SMs into a zeroed float32 buffer that the rotate-and-cache kernel consumes
                acc = ctx.workspace.get_zeroed("qkv_f32", (t, self.qkv_dim))
                ops.linear(h, self.w_qkv, acc, accumulate=True)
            else:
                ops.linear(h, self.w_qkv, qkv)
            if not fused:
                q = qkv[:, : self.q_dim].view(t, self.num_heads, self.head_dim)
                k = None if self.shares_cache else \
                    qkv[:, self.q_dim: self.q_dim + self.kv_dim].view(t, self.num_kv_heads, self.head_dim)
                pos.apply(ctx, q, k)
            ops.rope_kv_write(
                qkv, ctx.batch.positions,
                pos.cos if fused else None, pos.sin if fused else None, pos.rot_dim if fused else 0,
                self.num_heads, self.num_kv_heads, self.head_dim,
                cache.k, cache.v, kv_slots, src=acc)
        out = ctx.workspace.get("attn_out", (t, self.q_dim), ctx.dtype)
        ops.paged_attention(qkv, self.num_heads, self.num_kv_heads, self.head_dim, cache.k, cache.v,
                            cache.block_table, ctx.batch, out, self.scale, self.window, ctx.workspace)
        ops.linear(out, self.w_o, resid, accumulate=True)


register_part("mixer", "gqa_attention", GQAttention)
