"""A decode step as ONE kernel, where the model allows it.  An option (TLLM_FUSED_DECODE=1), off by
default: at the TinyLlama shape it measures 1.39 ms per step of eight requests against 0.82 ms for
the part-by-part path under a CUDA graph (its grid barriers and activation reloads cost what the
kernel boundaries cost there), so it is kept as a second, tested way to run the step, not the first.

When every request of a step brings one token (at most eight of them), every layer call is
RMSNorm -> grouped-query attention with rotary (or no) positions -> RMSNorm -> SwiGLU with the same
sizes, and the dtype is bfloat16, the runner can hand the step to `ops.decode_step` instead of
walking the parts: one persistent kernel streams all weights once through shared-memory rings.  The parts say themselves whether they can take part (`fused_decode()` returns
what the kernel needs from them, or None); a model with a part that cannot -- a mixer of another
kind, a layer that reads another layer's cache -- simply keeps the part-by-part path.  The result is
the same function of the weights and the cache, rounded at the same places.

The reference runs decode as one launch per operation and layer
(tiny_llm/runtime/cuda/cuda_runtime.cpp:658-802)."""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import ops


def enabled() -> bool:
    return os.environ.get("TLLM_FUSED_DECODE", "0") == "1"


class FusedDecode:
    def __init__(self, runner, layers, final_norm, head_dim: int, sizes: dict):
        self.runner = runner
        self.head_dim = head_dim
        self.sizes = sizes
        self.final_norm = final_norm
        self.layer_descs = layers          # keeps the tensors alive
        lib = ops.decode_step_library(head_dim)
        self.max_tokens = lib.tllm_decode_step_max_tokens()
        self.teams = lib.tllm_decode_step_teams()
        dev = runner.device
        table = (ops.DecodeLayer * len(layers))()
        for rec, (d, kv, group) in zip(table, layers):
            n1, mx, n2, ff = d
            rec.w_qkv, rec.w_o = mx["w_qkv"].data_ptr(), mx["w_o"].data_ptr()
            rec.w_gate_up, rec.w_down = ff["w_gate_up"].data_ptr(), ff["w_down"].data_ptr()
            rec.norm1, rec.norm2 = n1["weight"].data_ptr(), n2["weight"].data_ptr()
            rec.cos = 0 if mx["cos"] is None else mx["cos"].data_ptr()
            rec.sin = 0 if mx["sin"] is None else mx["sin"].data_ptr()
            rec.kcache, rec.vcache = kv[0].data_ptr(), kv[1].data_ptr()
            rec.block_table = runner._region(runner._dev_meta, f"block_table{group}").data_ptr()
            rec.slot_mapping = runner._region(runner._dev_meta, f"slot_mapping{group}").data_ptr()
            rec.eps1, rec.eps2 = n1["eps"], n2["eps"]
            rec.scale_log2 = mx["scale"] * math.log2(math.e)
            rec.window = int(mx["window"] or 0)
        raw = torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8)
        self.layer_table = raw.to(dev)
        self.sync_words = torch.zeros(4, dtype=torch.int64, device=dev)
        self.sm_count = torch.cuda.get_device_properties(dev).multi_processor_count

    # ---- does this model fit?
    @classmethod
    def build(cls, runner) -> Optional["FusedDecode"]:
        model, cache = runner.model, runner.cache
        if not enabled() or runner.dtype != torch.bfloat16 or runner.device.type != "cuda" or ops.force_generic:
            return None
        spec = model.spec
        layers = []
        sizes = None
        for pos, call in enumerate(spec.order):
            if call.reads_cache_of is not None:
                return None
            blk = model.blocks[call.layer]
            descs = []
            for part, kind in ((blk.norm1, "rms_norm"), (blk.mixer, "gqa_attention"), (blk.norm2, "rms_norm"),
                               (blk.ffn, "swiglu")):
                d = part.fused_decode() if hasattr(part, "fused_decode") else None
                if d is None or d["kind"] != kind:
                    return None
                descs.append(d)
            n1, mx, n2, ff = descs
            mine = {"hidden": mx["hidden_size"], "nq": mx["num_heads"], "nkv": mx["num_kv_heads"], "hd": mx["head_dim"],
                    "inter": ff["intermediate_size"], "block": ff["block"]}
            if n1["size"] != mine["hidden"] or n2["size"] != mine["hidden"] or ff["hidden_size"] != mine["hidden"]:
                return None
            if sizes is None:
                sizes = mine
            elif sizes != mine:
                return None     # the kernel has one set of sizes for all layers
            ref = cache.refs[pos]
            if ref.group is None:
                return None
            g = cache.groups[ref.group]
            if g.kv is None or not g.kv.is_contiguous() or g.kv.dtype != torch.bfloat16:
                return None
            layers.append((descs, (g.kv[ref.entry, 0], g.kv[ref.entry, 1]), ref.group))
        final = model.final_norm.fused_decode() if hasattr(model.final_norm, "fused_decode") else None
        if final is None or final["kind"] != "rms_norm" or sizes is None or final["size"] != sizes["hidden"]:
            return None
        if spec.hidden_size != sizes["hidden"] or sizes["hd"] % 16 or not 16 <= sizes["hd"] <= 256:
            return None
        probe = ops.DecodeParams()
        probe.n_layers, probe.m, probe.hidden, probe.nq, probe.nkv = len(layers), 1, sizes["hidden"], sizes["nq"], sizes["nkv"]
        probe.inter, probe.gu_block, probe.vocab = sizes["inter"], sizes["block"], spec.vocab_size
        probe.page_size, probe.max_blocks, probe.splits = cache.page_size, runner.max_blocks, 1
        if ops.decode_step_refusal(sizes["hd"], probe) is not None:
            return None
        return cls(runner, layers, final, sizes["hd"], sizes)

    def takes(self, batch) -> bool:
        return batch.max_q_len == 1 and batch.num_logits == batch.num_requests <= self.max_tokens

    def splits(self, m: int, max_kv_len: int) -> int:
        """Slices of keys per (request, key/value head): one item per attention team of the grid, each
        slice at least two 64-key tiles."""
        teams = self.sm_count * self.teams
        return max(1, min(teams // (m * self.sizes["nkv"]), (-(-max_kv_len // 64)) // 2, 32))

    def run(self, batch) -> torch.Tensor:
        """Logits [requests, vocab] of a step in which every request brings one token and wants its logits."""
        r, s, z = self.runner, self.runner.model.spec, self.sizes
        ws = r.workspace
        m = batch.num_requests
        q_dim = z["nq"] * z["hd"]
        splits = self.splits(m, batch.max_kv_len)
        p = ops.DecodeParams()
        p.layers = self.layer_table.data_ptr()
        p.tokens, p.positions, p.cu_q = batch.tokens.data_ptr(), batch.positions.data_ptr(), batch.cu_q.data_ptr()
        p.embed, p.final_norm, p.lm_head = r.model.embed.data_ptr(), self.final_norm["weight"].data_ptr(), r.model.lm_head.data_ptr()
        p.resid = ws.get("resid", (m, z["hidden"]), torch.float32).data_ptr()
        p.q_buf = ws.get("qkv", (m, q_dim + 2 * z["nkv"] * z["hd"]), torch.bfloat16).data_ptr()
        p.attn_out = ws.get("attn_out", (m, q_dim), torch.bfloat16).data_ptr()
        p.ffn_act = ws.get("ffn_act", (m, z["inter"]), torch.bfloat16).data_ptr()
        logits = ws.get("logits", (m, s.vocab_size), torch.float32)
        p.logits = logits.data_ptr()
        if splits > 1:
            part = ws.get("attention_partials", (m * z["nq"] * splits * (z["hd"] + 2),), torch.float32)
            p.part_o = part.data_ptr()
            p.part_ml = part.data_ptr() + m * z["nq"] * splits * z["hd"] * 4
        p.ssq_part = ws.get("norm_sums", (-(-z["hidden"] // 16), self.max_tokens), torch.float32).data_ptr()
        p.sync_words = self.sync_words.data_ptr()
        p.status = ops.status_word(r.device).data_ptr()
        p.n_layers, p.m, p.hidden, p.nq, p.nkv = len(self.layer_descs), m, z["hidden"], z["nq"], z["nkv"]
        p.inter, p.gu_block, p.vocab = z["inter"], z["block"], s.vocab_size
        p.page_size, p.max_blocks, p.splits = r.cache.page_size, r.max_blocks, splits
        p.final_eps = self.final_norm["eps"]
        ops.decode_step(self.head_dim, p)
        return logits
