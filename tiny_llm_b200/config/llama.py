"""Typed configuration of the Llama dense decoder, read from its own config.json keys.

Keys and their meaning follow tiny_llm/parser/llama_parser.cpp:164-276, which reads them from raw
JSON with no defaults; `eos_token_id` and `torch_dtype` follow tiny_llm/pipeline/pipeline.cpp:45-50,
80-82.  Differences, on purpose: `head_dim` and `tie_word_embeddings` are honoured (the reference
fixes head_dim = hidden_size / heads and always wants lm_head.weight), and a few keys have the
customary defaults listed in `_OPTIONAL`."""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Tuple

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

_REQUIRED_INT = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "max_position_embeddings")


def _get_int(d: dict, key: str, default=None) -> int:
    if key not in d or d[key] is None:
        if default is None:
            raise ConfigError(f'config.json: required key "{key}" is missing')
        return default
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f'config.json: key "{key}" must be a positive integer, found {v!r}')
    return v


def _get_float(d: dict, key: str, default=None) -> float:
    if key not in d or d[key] is None:
        if default is None:
            raise ConfigError(f'config.json: required key "{key}" is missing')
        return float(default)
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f'config.json: key "{key}" must be a positive number, found {v!r}')
    return float(v)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "float32"
    initializer_range: float = 0.02

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        # what the reference refuses (llama_parser.cpp:165-169), refused here by name
        if d.get("attention_bias", False):
            raise ConfigError('config.json: "attention_bias": true is not supported (no bias terms are built)')
        if d.get("mlp_bias", False):
            raise ConfigError('config.json: "mlp_bias": true is not supported (no bias terms are built)')
        if d.get("rope_scaling") is not None:
            raise ConfigError('config.json: "rope_scaling" must be null (scaled rotary tables are not built)')
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f'config.json: "hidden_act" must be "silu", found {act!r}')
        ints = {k: _get_int(d, k) for k in _REQUIRED_INT}
        nq = ints["num_attention_heads"]
        nkv = _get_int(d, "num_key_value_heads", default=nq)
        if nq % nkv != 0:
            raise ConfigError(f'config.json: "num_attention_heads" ({nq}) must be a multiple of '
                              f'"num_key_value_heads" ({nkv})')
        if "head_dim" in d and d["head_dim"] is not None:
            hd = _get_int(d, "head_dim")
        else:
            if ints["hidden_size"] % nq != 0:
                raise ConfigError(f'config.json: "hidden_size" ({ints["hidden_size"]}) is not a multiple of '
                                  f'"num_attention_heads" ({nq}) and no "head_dim" is given')
            hd = ints["hidden_size"] // nq
        if hd % 2 != 0:
            raise ConfigError(f'config.json: head_dim {hd} must be even for rotary position encoding')
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f'config.json: "eos_token_id" must be an integer, a list of integers or null, found {eos!r}')
        tie = d.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError(f'config.json: "tie_word_embeddings" must be true or false, found {tie!r}')
        dtype = d.get("torch_dtype", d.get("dtype", "float32"))
        if dtype not in ("float32", "bfloat16", "float16"):
            raise ConfigError(f'config.json: "torch_dtype" must be float32, bfloat16 or float16, found {dtype!r}')
        return cls(
            vocab_size=ints["vocab_size"], hidden_size=ints["hidden_size"],
            intermediate_size=ints["intermediate_size"], num_hidden_layers=ints["num_hidden_layers"],
            num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
            rms_norm_eps=_get_float(d, "rms_norm_eps"),
            rope_theta=_get_float(d, "rope_theta", default=10000.0),
            max_position_embeddings=ints["max_position_embeddings"],
            tie_word_embeddings=tie, eos_token_ids=eos_ids, torch_dtype=dtype,
            initializer_range=_get_float(d, "initializer_range", default=0.02))

    def to_dict(self) -> dict:
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        d.update(architectures=[self.architecture], model_type="llama", hidden_act="silu",
                 attention_bias=False, mlp_bias=False, rope_scaling=None)
        return d

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rotary", {"head_dim": self.head_dim, "theta": self.rope_theta,
                                   "max_positions": self.max_position_embeddings})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "position": rope, "window": None})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        layers = [LayerSpec(prefix=f"model.layers.{i}.", norm1=norm, mixer=mixer, norm2=norm, ffn=ffn)
                  for i in range(self.num_hidden_layers)]
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings, layers=layers,
            order=[LayerCall(i) for i in range(self.num_hidden_layers)], final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings, eos_token_ids=self.eos_token_ids,
            initializer_range=self.initializer_range,
            # older checkpoints store the rotary frequencies (the table here is made from rope_theta);
            # a tied model may still store its output matrix, which is the embedding table again
            ignored_weights=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if self.tie_word_embeddings else ()))


register_architecture(LlamaConfig.architecture, LlamaConfig)
