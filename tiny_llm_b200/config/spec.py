"""Architecture-neutral description of a decoder: which parts make up each layer and in which
order the layers run.  A configuration class turns its config.json keys into one `ModelSpec`;
the model builder reads nothing else, so no part ever learns which architecture it serves."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name from the part registry, with its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the parts it is made of and the kind of block that arranges them.

    `block` names an arrangement in the block registry.  The built-in "pre_norm" is
    x += mixer(norm1(x)); x += ffn(norm2(x)); other arrangements (post-norm, both branches from one
    normed input, norms on both sides of a part) are registered like parts and use the same fields,
    leaving out the ones they do not need and naming further parts in `more` as
    (role, family, PartSpec, weight name).  `prefix` is the weight-name prefix of the layer
    ("model.layers.3."); a part's weights are named prefix + its own name below."""
    prefix: str
    norm1: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    norm2: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    norm1_name: str = "input_layernorm"
    norm2_name: str = "post_attention_layernorm"
    block: str = "pre_norm"
    more: Tuple[Tuple[str, str, PartSpec, str], ...] = ()


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.  `layer` indexes `ModelSpec.layers` (a layer may be named
    twice).  Every call owns the cache entry with its own position in the order, unless
    `reads_cache_of` names an earlier call (by position in the order): then this call's mixer
    writes nothing and reads that call's cache."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: List[LayerSpec]
    order: List[LayerCall]
    final_norm: PartSpec
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    lm_head_name: str = "lm_head.weight"
    tie_word_embeddings: bool = False
    eos_token_ids: tuple = ()
    initializer_range: float = 0.02
    # name patterns of tensors that checkpoints of this architecture may carry and the model has no use for
    ignored_weights: tuple = ()
    # optional parts of family "hook" (forward(ctx, x) rewrites x in place): one on the float32 residual
    # right after the embedding (a scale, a learned position table), one on the float32 logits (a soft cap)
    after_embedding: Optional[PartSpec] = None
    on_logits: Optional[PartSpec] = None
    after_embedding_name: str = "model.after_embedding"
    on_logits_name: str = "model.on_logits"
