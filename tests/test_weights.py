"""Weights by name, the one error that lists everything, the safetensors container, random mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from tiny_llm_b200.config import LlamaConfig
from tiny_llm_b200.parts import DecoderModel
from tiny_llm_b200.weights import (FLOAT32, SafetensorsFile, WeightError, WeightSpec, load_state, random_state,
                                   save_safetensors, write_random_model)


def test_container_round_trip_and_library_agreement(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.randn(2, 2, 2).to(torch.float16)}
    ours = str(tmp_path / "ours.safetensors")
    save_safetensors(ours, t, metadata={"format": "pt"})
    with safe_open(ours, "pt") as f:          # the library reads what we wrote
        for k in t:
            assert torch.equal(f.get_tensor(k), t[k])
    theirs = str(tmp_path / "theirs.safetensors")
    save_file(t, theirs)
    f = SafetensorsFile(theirs)                # we read what the library wrote
    assert sorted(f.keys()) == sorted(t)
    for k in t:
        assert f.dtype(k) == t[k].dtype and f.shape(k) == tuple(t[k].shape) and torch.equal(f.get(k), t[k])
    f.close()


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFile(str(p))
    p = tmp_path / "len.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "off.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightError, match="data offsets"):
        SafetensorsFile(str(p))
    with pytest.raises(WeightError, match="no such"):
        SafetensorsFile(str(tmp_path / "none.safetensors"))


def test_names_shapes_and_fusions_of_the_model():
    model = DecoderModel(LlamaConfig.from_dict(TINY_A).model_spec())
    specs = model.weight_specs()
    assert specs["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert specs["model.layers.0.mlp.down_proj.weight"].shape == (64, 176)
    assert specs["model.norm.weight"].keep == FLOAT32 and "lm_head.weight" in specs
    assert len(specs) == 2 * 9 + 3
    tied = DecoderModel(LlamaConfig.from_dict(TINY_B).model_spec()).weight_specs()
    assert "lm_head.weight" not in tied


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_A)
    model = DecoderModel(cfg.model_spec())
    specs = model.weight_specs()
    state = random_state(specs, 0, 0.02, torch.float32)
    del state["model.layers.0.mlp.up_proj.weight"]
    del state["model.norm.weight"]
    state["model.layers.7.extra.weight"] = torch.zeros(2)
    state["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    state["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    path = str(tmp_path / "model.safetensors")
    save_safetensors(path, state)
    with pytest.raises(WeightError) as e:
        load_state(specs, str(tmp_path), torch.float32, "cpu")
    msg = str(e.value)
    for word in ("missing (2)", "model.layers.0.mlp.up_proj.weight", "model.norm.weight", "unexpected (1)",
                 "model.layers.7.extra.weight", "wrong shape or kind (2)", "expected shape [64, 64], found [64, 63]",
                 "model.embed_tokens.weight: expected floating point"):
        assert word in msg, (word, msg)


@pytest.mark.parametrize("stored", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("engine", [torch.float32, torch.bfloat16])
def test_kept_dtypes(tmp_path, stored, engine):
    cfg = LlamaConfig.from_dict(TINY_B)
    write_random_model(str(tmp_path), cfg, seed=3, dtype=stored)
    specs = DecoderModel(cfg.model_spec()).weight_specs()
    state = load_state(specs, str(tmp_path), engine, "cpu")
    assert state["model.layers.0.mlp.gate_proj.weight"].dtype == engine       # matrices: the engine's dtype
    assert state["model.layers.0.input_layernorm.weight"].dtype == torch.float32  # norm weights: always 32-bit
    as_stored = load_state({"model.norm.weight": WeightSpec("model.norm.weight", (96,), "as_stored")},
                           {"model.norm.weight": torch.ones(96, dtype=stored)}, engine, "cpu")
    assert as_stored["model.norm.weight"].dtype == (torch.float32 if stored == torch.float32 else engine)


def test_random_mode_is_seeded_and_writes_a_folder(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_A)
    a, b, c = (str(tmp_path / n) for n in "abc")
    write_random_model(a, cfg, seed=5)
    write_random_model(b, cfg, seed=5)
    write_random_model(c, cfg, seed=6)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    name = "model.layers.1.mlp.gate_proj.weight"
    assert torch.equal(fa.get(name), fb.get(name)) and not torch.equal(fa.get(name), fc.get(name))
    assert torch.equal(fa.get("model.norm.weight"), torch.ones(64))
    w = fa.get(name)
    assert abs(float(w.std()) - TINY_A["initializer_range"]) < 0.02 and abs(float(w.mean())) < 0.01
    from tiny_llm_b200.config import load_config
    assert load_config(a) == cfg


def test_gate_up_interleave():
    from tiny_llm_b200.parts import interleave_gate_up
    wg = torch.arange(12.).view(6, 2)
    wu = -torch.arange(12.).view(6, 2)
    f = interleave_gate_up(wg, wu, 2)
    assert torch.equal(f[0:2], wg[0:2]) and torch.equal(f[2:4], wu[0:2]) and torch.equal(f[8:10], wg[4:6])


def test_sharded_checkpoint_alias_of_the_output_matrix_and_harmless_extras(tmp_path):
    """A folder as large checkpoints are published: shards + index, no lm_head.weight (the embedding
    table stands in), and the rotary frequencies that older files carry."""
    from tiny_llm_b200.weights import ShardedSafetensors
    cfg = LlamaConfig.from_dict(TINY_A)
    spec = cfg.model_spec()
    specs = DecoderModel(spec).weight_specs()
    state = random_state(specs, 0, 0.02, torch.float32)
    whole = load_state(specs, state, torch.float32, "cpu")
    del state["lm_head.weight"]
    state["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    names = sorted(state)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fname, part in shards.items():
        save_safetensors(str(tmp_path / fname), {n: state[n] for n in part})
    index = {"metadata": {"total_size": 0}, "weight_map": {n: f for f, part in shards.items() for n in part}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_state(specs, str(tmp_path), torch.float32, "cpu", ignore=spec.ignored_weights)
    assert got["lm_head.weight"] is got["model.embed_tokens.weight"]          # one tensor, not a copy
    for n in specs:
        if n != "lm_head.weight":
            assert torch.equal(got[n], whole[n]), n
    # without the allow-list the extra tensor is an error, as every unknown tensor is
    with pytest.raises(WeightError, match=r"unexpected \(1\): model.layers.0.self_attn.rotary_emb.inv_freq"):
        load_state(specs, str(tmp_path), torch.float32, "cpu")
    # an index that names a tensor its shard does not hold, or a shard that is not there
    other = [f for f, part in shards.items() if "model.norm.weight" not in part][0]
    index["weight_map"]["model.norm.weight"] = other
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightError, match="is not in"):
        ShardedSafetensors(str(tmp_path))
    index["weight_map"]["model.norm.weight"] = "model-00003-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightError, match="no such weights file"):
        ShardedSafetensors(str(tmp_path))


def test_a_tied_model_tolerates_a_stored_output_matrix_and_an_untied_one_without_embedding_still_fails():
    cfg = LlamaConfig.from_dict(TINY_B)          # tied
    spec = cfg.model_spec()
    specs = DecoderModel(spec).weight_specs()
    state = random_state(specs, 1, 0.02, torch.float32)
    state["lm_head.weight"] = state["model.embed_tokens.weight"].clone()
    assert "lm_head.weight" not in load_state(specs, state, torch.float32, "cpu", ignore=spec.ignored_weights)
    untied = DecoderModel(LlamaConfig.from_dict(TINY_A).model_spec()).weight_specs()
    st = random_state(untied, 0, 0.02, torch.float32)
    del st["lm_head.weight"], st["model.embed_tokens.weight"]
    with pytest.raises(WeightError, match=r"missing \(2\): lm_head.weight, model.embed_tokens.weight"):
        load_state(untied, st, torch.float32, "cpu")
