"""Another arrangement of a layer, defined here and never part of the framework: one normed input
feeds the mixer and the feed-forward side by side, their summed branch is normed again and only then
joins the residual stream (a "parallel residual" with a norm on both sides).  Around the layers, two
toy hooks: the embedding scaled by a constant, the logits soft-capped.  The block and the hooks are
registered from this file, named by the spec, loaded by tensor name and stepped in portions and single
tokens -- without a change to the framework's files."""
import math

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WIDTH, HEADS, KV, HD, INNER, VOCAB, MAXPOS = 48, 3, 1, 16, 80, 97, 96
CAP = 3.0


class ParallelSandwichBlock:
    """x += post(mixer(pre(x)) + ffn(pre(x))).  The parts add into whatever float32 buffer they are
    given, so the branch is a zeroed scratch buffer instead of the residual stream."""

    def __init__(self, spec, shares_cache=False):
        from tiny_llm_b200.parts import build_part
        assert spec.norm2 is None and len(spec.more) == 1 and spec.more[0][0] == "post"
        self.spec = spec
        self.pre = build_part("norm", spec.norm1)
        self.mixer = build_part("mixer", spec.mixer)
        self.ffn = build_part("ffn", spec.ffn)
        _, family, post_spec, self.post_name = spec.more[0]
        self.post = build_part(family, post_spec)

    def parts(self):
        return [self.pre, self.mixer, self.ffn, self.post]

    def _names(self):
        p = self.spec.prefix
        return p + self.spec.norm1_name, p + self.spec.mixer_prefix, p + self.spec.ffn_prefix, p + self.post_name

    def weight_specs(self):
        a, b, c, d = self._names()
        return self.pre.weight_specs(a) + self.mixer.weight_specs(b) + self.ffn.weight_specs(c) + self.post.weight_specs(d)

    def load(self, weights):
        a, b, c, d = self._names()
        self.pre.load(a, weights), self.mixer.load(b, weights), self.ffn.load(c, weights), self.post.load(d, weights)

    def forward(self, ctx, resid, cache):
        h = self.pre.forward(ctx, resid)
        h = ctx.workspace.get("toy_pre_out", h.shape, h.dtype).copy_(h)   # the post norm reuses the norm's buffer
        branch = ctx.workspace.get("toy_branch", resid.shape, torch.float32).zero_()
        self.mixer.forward(ctx, h, branch, cache)
        self.ffn.forward(ctx, h, branch)
        resid += self.post.forward(ctx, branch).float()


class EmbeddingScale:
    def __init__(self, factor):
        self.factor = float(factor)

    def weight_specs(self, prefix):
        return []

    def load(self, prefix, weights):
        pass

    def forward(self, ctx, x):
        x.mul_(self.factor)


class SoftCap:
    def __init__(self, cap):
        self.cap = float(cap)

    def weight_specs(self, prefix):
        return []

    def load(self, prefix, weights):
        pass

    def forward(self, ctx, x):
        x.copy_(self.cap * torch.tanh(x / self.cap))


def toy_spec():
    from tiny_llm_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec
    norm = PartSpec("rms_norm", {"size": WIDTH, "eps": 1e-5})
    rope = PartSpec("rotary", {"head_dim": HD, "theta": 100.0, "max_positions": MAXPOS})
    attn = PartSpec("gqa_attention", {"hidden_size": WIDTH, "num_heads": HEADS, "num_kv_heads": KV, "head_dim": HD,
                                      "position": rope, "window": None})
    ffn = PartSpec("swiglu", {"hidden_size": WIDTH, "intermediate_size": INNER})
    toy = LayerSpec("model.layers.0.", norm1=norm, mixer=attn, ffn=ffn, block="parallel_sandwich",
                    more=(("post", "norm", norm, "post_branch_layernorm"),))
    plain = LayerSpec("model.layers.1.", norm, attn, norm, ffn)       # the framework's own block beside it
    return ModelSpec("ToyBlockForCausalLM", VOCAB, WIDTH, MAXPOS, [toy, plain], [LayerCall(0), LayerCall(1)], norm,
                     initializer_range=0.2,
                     after_embedding=PartSpec("embedding_scale", {"factor": math.sqrt(WIDTH)}),
                     on_logits=PartSpec("soft_cap", {"cap": CAP}))


def plain_toy(w, toks):
    t = len(toks)
    pos = torch.arange(t)
    c = {"num_attention_heads": HEADS, "num_key_value_heads": KV, "head_dim": HD, "hidden_size": WIDTH}
    cos, sin = pl.rope_tables(MAXPOS, HD, 100.0)
    x = pl.embedding(w["model.embed_tokens.weight"], torch.tensor(toks)) * math.sqrt(WIDTH)
    p = "model.layers.0."
    h = pl.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
    branch = pl.attention_block(h, w, p + "self_attn.", c, cos, sin, pos) + \
        pl.swiglu_mlp(h, *(w[p + f"mlp.{n}_proj.weight"] for n in ("gate", "up", "down")))
    x = x + pl.rms_norm(branch, w[p + "post_branch_layernorm.weight"], 1e-5)
    p = "model.layers.1."
    h = pl.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
    x = x + pl.attention_block(h, w, p + "self_attn.", c, cos, sin, pos)
    h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
    x = x + pl.swiglu_mlp(h, *(w[p + f"mlp.{n}_proj.weight"] for n in ("gate", "up", "down")))
    logits = pl.linear(pl.rms_norm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"])
    return CAP * torch.tanh(logits / CAP)


def test_another_block_arrangement_and_hooks_around_the_layers():
    from tiny_llm_b200.engine import StepEntry, make_runner
    from tiny_llm_b200.parts import DecoderModel, register_block, register_part, registered_blocks
    from tiny_llm_b200.weights import load_state, random_state

    register_block("parallel_sandwich", ParallelSandwichBlock)
    register_part("hook", "embedding_scale", EmbeddingScale)
    register_part("hook", "soft_cap", SoftCap)
    assert {"pre_norm", "parallel_sandwich"} <= set(registered_blocks())
    model = DecoderModel(toy_spec())
    specs = model.weight_specs()
    assert "model.layers.0.post_branch_layernorm.weight" in specs
    assert "model.layers.0.post_attention_layernorm.weight" not in specs
    assert not model.graph_safe      # the toy hooks compute with torch: steps of this model are not captured
    state = random_state(specs, 9, 0.2, torch.float32)
    # a post norm that is not all ones, so that leaving it out or putting it elsewhere shows
    state["model.layers.0.post_branch_layernorm.weight"] = torch.linspace(0.5, 1.5, WIDTH)
    model.load(load_state(specs, state, torch.float32, DEV))
    runner = make_runner(model, "float32", DEV, max_tokens=128, page_size=8, max_requests=2)
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, VOCAB, (41,), generator=g).tolist()
    b = torch.randint(0, VOCAB, (9,), generator=g).tolist()
    ref_a, ref_b = plain_toy(state, a), plain_toy(state, b)
    assert float(ref_a.abs().max()) > 0.5 * CAP      # the cap bites: logits without it would be larger
    runner.cache.add_request("a"), runner.cache.add_request("b")
    got_a, got_b = [], []
    plan = [((0, 17), (0, 2)), ((17, 18), (2, 3)), ((18, 20), (3, 4)), ((20, 40), (4, 9)), ((40, 41), None)]
    for ra, rb in plan:
        entries = [StepEntry("a", a[ra[0]:ra[1]], range(ra[1] - ra[0]))]
        if rb:
            entries.append(StepEntry("b", b[rb[0]:rb[1]], range(rb[1] - rb[0])))
        out = runner.step(entries).cpu()
        got_a.append(out[: ra[1] - ra[0]].clone())
        if rb:
            got_b.append(out[ra[1] - ra[0]:].clone())
    assert float((torch.cat(got_a) - ref_a).abs().max()) < 2e-5
    assert float((torch.cat(got_b) - ref_b).abs().max()) < 2e-5


def test_an_unknown_block_kind_is_named():
    from tiny_llm_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec
    from tiny_llm_b200.parts import DecoderModel
    norm = PartSpec("rms_norm", {"size": 8, "eps": 1e-5})
    spec = ModelSpec("X", 10, 8, 16, [LayerSpec("l.", norm1=norm, block="no_such_block")], [LayerCall(0)], norm)
    with pytest.raises(KeyError, match="no_such_block"):
        DecoderModel(spec)
