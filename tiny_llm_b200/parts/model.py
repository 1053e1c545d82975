"""The decoder put together from parts: embedding (and the spec's hook after it), the layer calls of
`ModelSpec.order`, final norm on the wanted rows only, LM head in 32-bit logits (and the spec's hook on
them).  How one layer arranges its parts is a registered block kind named by the layer's spec
("pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x))), and the run order is a list of the spec; the
reference hard-codes both in its parser (tiny_llm/parser/llama_parser.cpp:181-271)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.spec import LayerSpec, ModelSpec
from ..weights import COMPUTE, WeightSpec
from .registry import build_block, build_part, register_block


class Block:
    """The pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))."""

    def __init__(self, spec: LayerSpec, shares_cache: bool = False):
        for role in ("norm1", "mixer", "norm2", "ffn"):
            if getattr(spec, role) is None:
                raise ValueError(f"layer {spec.prefix!r}: a pre_norm block needs a {role}")
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1)
        self.norm2 = build_part("norm", spec.norm2)
        self.mixer = build_part("mixer", spec.mixer, **({"shares_cache": True} if shares_cache else {}))
        self.ffn = build_part("ffn", spec.ffn)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def _prefixes(self):
        p = self.spec.prefix
        return p + self.spec.norm1_name, p + self.spec.mixer_prefix, p + self.spec.norm2_name, p + self.spec.ffn_prefix

    def weight_specs(self) -> List[WeightSpec]:
        n1, mx, n2, ff = self._prefixes()
        return (self.norm1.weight_specs(n1) + self.mixer.weight_specs(mx) +
                self.norm2.weight_specs(n2) + self.ffn.weight_specs(ff))

    def load(self, weights) -> None:
        n1, mx, n2, ff = self._prefixes()
        self.norm1.load(n1, weights)
        self.mixer.load(mx, weights)
        self.norm2.load(n2, weights)
        self.ffn.load(ff, weights)

    def forward(self, ctx, resid, cache) -> None:
        h = self.norm1.forward(ctx, resid)
        self.mixer.forward(ctx, h, resid, cache)
        h = self.norm2.forward(ctx, resid)
        self.ffn.forward(ctx, h, resid)


register_block("pre_norm", Block)


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        for pos, call in enumerate(spec.order):
            if not 0 <= call.layer < len(spec.layers):
                raise ValueError(f"run order entry {pos} names layer {call.layer}, the model has {len(spec.layers)}")
            if call.reads_cache_of is not None and not 0 <= call.reads_cache_of < pos:
                raise ValueError(f"run order entry {pos} reads the cache of entry {call.reads_cache_of}, "
                                 f"which does not run before it")
        shared = {c.layer for c in spec.order if c.reads_cache_of is not None}
        owning = {c.layer for c in spec.order if c.reads_cache_of is None}
        if shared & owning:
            raise ValueError(f"layers {sorted(shared & owning)} are run both with a cache of their own and with another's")
        self.blocks = [build_block(ls, shares_cache=(i in shared)) for i, ls in enumerate(spec.layers)]
        self.final_norm = build_part("norm", spec.final_norm)
        self.after_embedding = None if spec.after_embedding is None else build_part("hook", spec.after_embedding)
        self.on_logits = None if spec.on_logits is None else build_part("hook", spec.on_logits)
        self.embed = None
        self.lm_head = None
        self.loaded = False
        # a part that synchronises or computes on the host must not be captured; parts say so themselves
        parts = [self.final_norm] + [x for b in self.blocks for x in b.parts()] + \
            [h for h in (self.after_embedding, self.on_logits) if h is not None]
        self.graph_safe = all(getattr(x, "graph_safe", False) for x in parts)

    # ---- what the model wants from the weights and the cache
    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = self.spec
        specs = [WeightSpec(s.embed_name, (s.vocab_size, s.hidden_size), COMPUTE)]
        for b in self.blocks:
            specs += b.weight_specs()
        specs += self.final_norm.weight_specs(s.final_norm_name)
        if self.after_embedding is not None:
            specs += self.after_embedding.weight_specs(s.after_embedding_name)
        if self.on_logits is not None:
            specs += self.on_logits.weight_specs(s.on_logits_name)
        if not s.tie_word_embeddings:
            # a checkpoint without an output matrix uses the embedding table for it
            specs.append(WeightSpec(s.lm_head_name, (s.vocab_size, s.hidden_size), COMPUTE, alias_of=s.embed_name))
        out = {}
        for w in specs:
            if w.name in out and out[w.name] != w:
                raise ValueError(f"two parts want tensor {w.name!r} with different shapes")
            out[w.name] = w
        return out

    def cache_needs(self):
        """One need per run-order entry; None for an entry that reads another entry's cache or needs none."""
        def need(block):
            return None if block.mixer is None else block.mixer.cache_need()
        return [None if c.reads_cache_of is not None else need(self.blocks[c.layer]) for c in self.spec.order]

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed = weights[s.embed_name]
        for b in self.blocks:
            b.load(weights)
        self.final_norm.load(s.final_norm_name, weights)
        if self.after_embedding is not None:
            self.after_embedding.load(s.after_embedding_name, weights)
        if self.on_logits is not None:
            self.on_logits.load(s.on_logits_name, weights)
        self.lm_head = self.embed if s.tie_word_embeddings else weights[s.lm_head_name]
        self.loaded = True

    # ---- one step
    def forward(self, ctx) -> torch.Tensor:
        """Runs the step's tokens through every layer call; returns float32 logits at
        `ctx.batch.logit_rows` ([n_out, vocab]), or None when no row is wanted."""
        s = self.spec
        b = ctx.batch
        resid = ctx.workspace.get("resid", (b.num_tokens, s.hidden_size), torch.float32)
        ops.embedding(b.tokens, self.embed, resid)
        if self.after_embedding is not None:
            self.after_embedding.forward(ctx, resid)
        for pos, call in enumerate(s.order):
            owner = pos if call.reads_cache_of is None else call.reads_cache_of
            self.blocks[call.layer].forward(ctx, resid, ctx.cache_view(owner))
        if b.num_logits == 0:
            return None
        h = self.final_norm.forward(ctx, resid, rows=b.logit_rows)
        logits = ctx.workspace.get("logits", (b.num_logits, s.vocab_size), torch.float32)
        ops.linear(h, self.lm_head, logits)
        if self.on_logits is not None:
            self.on_logits.forward(ctx, logits)
        return logits
