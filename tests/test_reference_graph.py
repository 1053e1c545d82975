"""The graph that zscey/tiny-llm's own parser builds (tiny_llm/parser/llama_parser.cpp:164-276), walked on the
host: which tensors it wants by name and shape, which ops it runs in which order and how they are wired.
Checked against it: the weights `DecoderModel.weight_specs()` declares, and the order in which
`plain_llama.forward` composes its parts.  Needs the reference arm's binary (baseline/build_reference.py builds
it from the reference's unmodified sources; `ref_driver graph` needs no GPU); skipped where it has not been built."""
import json
import os
import subprocess

import pytest

from conftest import TINY_A, TINY_B
from tiny_llm_b200.config import LlamaConfig
from tiny_llm_b200.parts import DecoderModel

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "baseline", "_ref", "ref_driver")
TINYLLAMA = dict(TINY_A, num_hidden_layers=22, hidden_size=2048, num_attention_heads=32, num_key_value_heads=4,
                 intermediate_size=5632, vocab_size=32000, max_position_embeddings=2048)

pytestmark = pytest.mark.skipif(not os.path.isfile(DRIVER), reason="the reference arm has not been built here")


def reference_graph(cfg: dict, tmp_path):
    c = dict(cfg)
    if not isinstance(c.get("eos_token_id"), int):
        c["eos_token_id"] = None            # the reference reads one integer or null
    path = tmp_path / "config.json"
    path.write_text(json.dumps(c))
    res = subprocess.run([DRIVER, "graph", "--config", str(path)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr
    return json.loads(res.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINYLLAMA], ids=["A", "B", "tinyllama"])
def test_the_reference_wants_the_tensors_the_model_declares(cfg, tmp_path):
    g = reference_graph(cfg, tmp_path)
    assert g["valid"] and sorted(g["inputs"]) == ["pos_ids", "token_ids"] and g["outputs"] == ["lm_head.out"]
    theirs = {k: tuple(v) for k, v in g["sources"].items() if k not in g["inputs"]}
    ours = {n: tuple(s.shape) for n, s in DecoderModel(LlamaConfig.from_dict(cfg).model_spec()).weight_specs().items()}
    if cfg.get("tie_word_embeddings"):
        # the reference never ties (llama_parser.cpp:264-271 always declares lm_head.weight); here the table stands in
        assert theirs.pop("lm_head.weight") == ours["model.embed_tokens.weight"]
    assert theirs == ours


def test_the_reference_runs_the_parts_in_the_order_of_the_plain_implementation(tmp_path):
    """plain_llama.forward: embedding; per layer norm -> attention -> residual -> norm -> gate, SiLU, up, product,
    down -> residual; final norm; output matrix.  The reference's nodes, in its own order and wiring."""
    g = reference_graph(TINY_A, tmp_path)
    nodes = g["nodes"]
    layers = TINY_A["num_hidden_layers"]
    assert [n["kind"] for n in nodes[:2]] == ["embedding", "rope"]
    assert [n["kind"] for n in nodes[-2:]] == ["rms_norm", "slice_linear"] and len(nodes) == 2 + 10 * layers + 2
    stream = "model.embed_tokens.out"                       # the residual stream as the layer finds it
    for i in range(layers):
        p = f"model.layers.{i}."
        n = {x["name"][len(p):]: x for x in nodes[2 + 10 * i: 12 + 10 * i]}
        assert [x["kind"] for x in nodes[2 + 10 * i: 12 + 10 * i]] == \
            ["rms_norm", "causal_attention", "add", "rms_norm", "linear", "silu", "linear", "mul", "linear", "add"]
        assert n["input_layernorm"]["inputs"] == [stream, p + "input_layernorm.weight"]
        att = n["self_attn"]["inputs"]
        assert att[0] == p + "input_layernorm.out" and att[1:4] == ["rope.cos", "rope.sin", "pos_ids"]
        assert att[4:] == [p + f"self_attn.{w}_proj.weight" for w in "qkvo"]
        assert n["attn_residual"]["inputs"] == [stream, p + "self_attn.out"]                  # x1 = x + attention(norm(x))
        assert n["post_attention_layernorm"]["inputs"][0] == p + "attn_residual.out"
        normed = p + "post_attention_layernorm.out"
        assert n["mlp.gate_proj"]["inputs"][0] == normed and n["mlp.up_proj"]["inputs"][0] == normed
        assert n["mlp.act"]["inputs"] == [p + "mlp.gate_proj.out"]                            # SiLU on the gate
        assert n["mlp.mul"]["inputs"] == [p + "mlp.act.out", p + "mlp.up_proj.out"]
        assert n["mlp.down_proj"]["inputs"][0] == p + "mlp.mul.out"
        assert n["mlp_residual"]["inputs"] == [p + "attn_residual.out", p + "mlp.down_proj.out"]   # x = x1 + mlp(norm(x1))
        stream = p + "mlp_residual.out"
    assert nodes[-2]["inputs"] == [stream, "model.norm.weight"]
    assert nodes[-1]["inputs"] == ["model.norm.out", "lm_head.weight"]
