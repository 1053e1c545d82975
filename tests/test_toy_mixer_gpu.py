"""A toy mixer with state of its own, defined here, is registered, built and stepped without a
change to the framework's files: a new architecture name, a configuration class that maps its
config.json keys to a ModelSpec, and a mixer part that declares a StateNeed.  Its model mixes
mixers: layer 0 uses the toy, layer 1 grouped-query attention."""
import json
from dataclasses import dataclass

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class DecayingSum:
    """state_t = decay * state_{t-1} + h_t (32-bit, per request); out_t = state_t W^T."""

    def __init__(self, hidden_size: int, decay: float, shares_cache: bool = False):
        self.hidden_size, self.decay, self.w = hidden_size, decay, None

    def cache_need(self):
        from tiny_llm_b200.cache import StateNeed
        return StateNeed((self.hidden_size,), torch.float32)

    def weight_specs(self, prefix):
        from tiny_llm_b200.weights import WeightSpec
        return [WeightSpec(prefix + "mix.weight", (self.hidden_size, self.hidden_size))]

    def load(self, prefix, weights):
        self.w = weights[prefix + "mix.weight"]

    def forward(self, ctx, h, resid, cache):
        b = ctx.batch
        slots = b.slots.tolist()
        start = 0
        for slot, n in zip(slots, b.host_q_lens):
            s = cache.state[slot]
            for t in range(start, start + n):
                s = self.decay * s + h[t].float()
                resid[t] += s @ self.w.float().t()
            cache.state[slot] = s
            start += n


@dataclass(frozen=True)
class ToyConfig:
    vocab: int
    width: int
    inner: int
    decay: float
    eps: float
    positions: int
    architecture = "ToyStateForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab"], d["width"], d["inner"], d["decay"], d["eps"], d["positions"])

    def to_dict(self):
        return dict(architectures=[self.architecture], vocab=self.vocab, width=self.width, inner=self.inner,
                    decay=self.decay, eps=self.eps, positions=self.positions)

    def model_spec(self):
        from tiny_llm_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.eps})
        ffn = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": self.inner})
        toy = PartSpec("decaying_sum", {"hidden_size": self.width, "decay": self.decay})
        rope = PartSpec("rotary", {"head_dim": 16, "theta": 100.0, "max_positions": self.positions})
        attn = PartSpec("gqa_attention", {"hidden_size": self.width, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                          "position": rope, "window": None})
        layers = [LayerSpec("model.layers.0.", norm, toy, norm, ffn, mixer_prefix="toy."),
                  LayerSpec("model.layers.1.", norm, attn, norm, ffn)]
        return ModelSpec(self.architecture, self.vocab, self.width, self.positions, layers,
                         [LayerCall(0), LayerCall(1)], norm, initializer_range=0.2)


def plain_toy(cfg, w, toks):
    x = pl.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    t = len(toks)
    # layer 0: the toy
    h = pl.rms_norm(x, w["model.layers.0.input_layernorm.weight"], cfg.eps)
    s = torch.zeros(cfg.width)
    out = []
    for i in range(t):
        s = cfg.decay * s + h[i]
        out.append(s @ w["model.layers.0.toy.mix.weight"].t())
    x = x + torch.stack(out)
    h = pl.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], cfg.eps)
    x = x + pl.swiglu_mlp(h, *(w[f"model.layers.0.mlp.{n}_proj.weight"] for n in ("gate", "up", "down")))
    # layer 1: attention
    c = {"num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16, "hidden_size": cfg.width}
    cos, sin = pl.rope_tables(cfg.positions, 16, 100.0)
    h = pl.rms_norm(x, w["model.layers.1.input_layernorm.weight"], cfg.eps)
    x = x + pl.attention_block(h, w, "model.layers.1.self_attn.", c, cos, sin, torch.arange(t))
    h = pl.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], cfg.eps)
    x = x + pl.swiglu_mlp(h, *(w[f"model.layers.1.mlp.{n}_proj.weight"] for n in ("gate", "up", "down")))
    return pl.linear(pl.rms_norm(x, w["model.norm.weight"], cfg.eps), w["lm_head.weight"])


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    from tiny_llm_b200.config import load_config, register_architecture
    from tiny_llm_b200.engine import StepEntry, load_model, make_runner
    from tiny_llm_b200.parts import register_part
    from tiny_llm_b200.weights import write_random_model

    register_part("mixer", "decaying_sum", DecayingSum)
    register_architecture(ToyConfig.architecture, ToyConfig)
    cfg = ToyConfig(vocab=97, width=48, inner=80, decay=0.75, eps=1e-5, positions=64)
    write_random_model(str(tmp_path), cfg, seed=3)
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["ToyStateForCausalLM"]
    assert load_config(str(tmp_path)) == cfg
    _, model = load_model(str(tmp_path), "float32", DEV)
    runner = make_runner(model, "float32", DEV, max_tokens=128, page_size=8, max_requests=2)
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].num_entries == 1
    assert runner.cache.refs[0].state == 0 and runner.cache.refs[1].group == 0
    w = pl.load_weights(str(tmp_path))
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 97, (30,), generator=g).tolist()
    b = torch.randint(0, 97, (21,), generator=g).tolist()
    ref_a, ref_b = plain_toy(cfg, w, a), plain_toy(cfg, w, b)
    cache = runner.cache
    cache.add_request("a"), cache.add_request("b")
    got_a, got_b = [], []
    plan = [((0, 7), (0, 2)), ((7, 8), (2, 13)), ((8, 20), None), ((20, 21), (13, 14)), ((21, 30), (14, 21))]
    for ra, rb in plan:
        entries = [StepEntry("a", a[ra[0]:ra[1]], range(ra[1] - ra[0]))]
        if rb:
            entries.append(StepEntry("b", b[rb[0]:rb[1]], range(rb[1] - rb[0])))
        out = runner.step(entries).cpu()
        got_a.append(out[: ra[1] - ra[0]].clone())
        if rb:
            got_b.append(out[ra[1] - ra[0]:].clone())
    assert float((torch.cat(got_a) - ref_a).abs().max()) < 2e-5 * max(1.0, float(ref_a.abs().max()))
    assert float((torch.cat(got_b) - ref_b).abs().max()) < 2e-5 * max(1.0, float(ref_b.abs().max()))
    # a slot that is handed out again starts from a zero state
    cache.free_request("a")
    cache.add_request("c")
    out = runner.step([StepEntry("c", a, range(30))]).cpu()
    assert float((out - ref_a).abs().max()) < 2e-5 * max(1.0, float(ref_a.abs().max()))
