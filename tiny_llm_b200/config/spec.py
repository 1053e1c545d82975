"""Architecture-neutral description of a decoder: which parts make up each layer and in which
order the layers run.  A configuration class turns its config.json keys into one `ModelSpec`;
the model builder reads nothing else, so no part ever learns which architecture it serves."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name from the part registry, with its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x)).
    `prefix` is the weight-name prefix of the layer ("model.layers.3.")."""
    prefix: str
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    norm1_name: str = "input_layernorm"
    norm2_name: str = "post_attention_layernorm"


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
