"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from tiny_llm_b200.config import (ConfigError, LlamaConfig, config_from_dict, load_config, register_architecture,
                                  registered_architectures)


def test_reads_every_size_from_its_keys():
    a = LlamaConfig.from_dict(TINY_A)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.max_position_embeddings) == (2, 64, 4, 2, 16, 176, 256, 128)
    assert a.rope_theta == 10000.0 and a.rms_norm_eps == 1e-5 and not a.tie_word_embeddings
    assert a.eos_token_ids == (2,)
    b = LlamaConfig.from_dict(TINY_B)
    assert b.head_dim == 32 and b.num_key_value_heads == 1 and b.tie_word_embeddings
    assert b.eos_token_ids == (5, 7) and b.rope_theta == 500000.0 and b.rms_norm_eps == 1e-6
    c = LlamaConfig.from_dict(TINY_C)
    assert c.head_dim == 48 and c.head_dim * c.num_attention_heads != c.hidden_size


def test_defaults_and_round_trip():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "rope_theta", "eos_token_id")}
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads and c.rope_theta == 10000.0 and c.eos_token_ids == ()
    again = config_from_dict(LlamaConfig.from_dict(TINY_B).to_dict())
    assert again == LlamaConfig.from_dict(TINY_B)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "max_position_embeddings", "rms_norm_eps"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"attention_bias": True}, "attention_bias"), ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"hidden_size": 66}, "head_dim"),
    ({"vocab_size": -1}, "vocab_size"), ({"vocab_size": "big"}, "vocab_size"), ({"eos_token_id": "x"}, "eos_token_id"),
    ({"torch_dtype": "int8"}, "torch_dtype"), ({"head_dim": 15}, "head_dim")])
def test_refused_values_name_their_key(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(d)


def test_registry_picks_by_architecture_name(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="NoSuchForCausalLM.*LlamaForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["NoSuchForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path)) == LlamaConfig.from_dict(TINY_B)
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nowhere"))
    with pytest.raises(TypeError):
        register_architecture("Broken", object)


def test_model_spec_is_data():
    spec = LlamaConfig.from_dict(TINY_B).model_spec()
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2]
    lay = spec.layers[1]
    assert lay.mixer.kind == "gqa_attention" and lay.ffn.kind == "swiglu" and lay.norm1.kind == "rms_norm"
    assert lay.mixer.params["num_kv_heads"] == 1 and lay.mixer.params["position"].params["theta"] == 500000.0
    assert lay.norm1.params["eps"] == 1e-6 and lay.ffn.params["intermediate_size"] == 256
    assert spec.tie_word_embeddings and spec.eos_token_ids == (5, 7)
