"""Two more toy parts, defined here and never part of the framework: a feed-forward that routes
every token to one of its experts, and a position encoding of another kind (it scales queries and
keys by position instead of rotating them).  They are registered, put into a model by spec beside
the framework's own parts (layer 0: rotary attention + routed feed-forward; layer 1: scaled
attention + SwiGLU), loaded by tensor name and stepped in portions and single tokens -- without a
change to the framework's files."""
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class RoutedFeedForward:
    """m = W_down[e] relu(W_up[e] y) with e = argmax(router y): one expert per token."""

    def __init__(self, hidden_size: int, inner_size: int, experts: int):
        self.h, self.i, self.e = hidden_size, inner_size, experts
        self.router = self.up = self.down = None

    def weight_specs(self, prefix):
        from tiny_llm_b200.weights import FLOAT32, WeightSpec
        return [WeightSpec(prefix + "router.weight", (self.e, self.h), FLOAT32),
                WeightSpec(prefix + "experts.up", (self.e, self.i, self.h)),
                WeightSpec(prefix + "experts.down", (self.e, self.h, self.i))]

    def load(self, prefix, weights):
        self.router, self.up, self.down = (weights[prefix + n] for n in ("router.weight", "experts.up", "experts.down"))

    def forward(self, ctx, h, resid):
        y = h.float()
        choice = (y @ self.router.t()).argmax(dim=1)          # router logits in 32-bit
        for e in range(self.e):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                z = torch.relu(y[rows] @ self.up[e].float().t())
                resid[rows] += z @ self.down[e].float().t()


class PositionScale:
    """q, k of the token at position p are multiplied by 1 + p / span (not a rotation: the mixer calls
    `apply` on its query and key views instead of handing tables to its fused kernel)."""
    fused = False
    cos = sin = None
    rot_dim = 0

    def __init__(self, span: float):
        self.span = float(span)

    def prepare(self, device):
        pass

    def apply(self, ctx, q, k):
        f = (1.0 + ctx.batch.positions.float() / self.span)[:, None, None]
        q.copy_((q.float() * f).to(q.dtype))
        if k is not None:
            k.copy_((k.float() * f).to(k.dtype))


def toy_spec():
    from tiny_llm_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec
    width, heads, kv, hd = 48, 3, 1, 16
    norm = PartSpec("rms_norm", {"size": width, "eps": 1e-5})
    rope = PartSpec("rotary", {"head_dim": hd, "theta": 100.0, "max_positions": 96})
    scale = PartSpec("position_scale", {"span": 40.0})
    attn = lambda pos: PartSpec("gqa_attention", {"hidden_size": width, "num_heads": heads, "num_kv_heads": kv,
                                                  "head_dim": hd, "position": pos, "window": None})
    routed = PartSpec("routed_relu", {"hidden_size": width, "inner_size": 40, "experts": 3})
    swiglu = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": 80})
    layers = [LayerSpec("model.layers.0.", norm, attn(rope), norm, routed, ffn_prefix="moe."),
              LayerSpec("model.layers.1.", norm, attn(scale), norm, swiglu)]
    return ModelSpec("ToyPartsForCausalLM", 101, width, 96, layers, [LayerCall(0), LayerCall(1)], norm,
                     initializer_range=0.2)


def plain_toy(w, toks):
    t = len(toks)
    pos = torch.arange(t)
    c = {"num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "hidden_size": 48}
    x = pl.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    # layer 0: rotary attention, routed feed-forward
    cos, sin = pl.rope_tables(96, 16, 100.0)
    h = pl.rms_norm(x, w["model.layers.0.input_layernorm.weight"], 1e-5)
    x = x + pl.attention_block(h, w, "model.layers.0.self_attn.", c, cos, sin, pos)
    h = pl.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-5)
    logits = h @ w["model.layers.0.moe.router.weight"].t()
    choice = logits.argmax(dim=1)
    top2 = logits.topk(2, dim=1).values
    assert float((top2[:, 0] - top2[:, 1]).min()) > 1e-3    # no token on the fence, where rounding could flip the choice
    out = torch.zeros_like(x)
    for i in range(t):
        e = int(choice[i])
        out[i] = torch.relu(h[i] @ w["model.layers.0.moe.experts.up"][e].t()) @ w["model.layers.0.moe.experts.down"][e].t()
    x = x + out
    # layer 1: queries and keys scaled by position, SwiGLU
    p = "model.layers.1.self_attn."
    h = pl.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-5)
    f = (1.0 + pos.float() / 40.0)[:, None, None]
    q = pl.linear(h, w[p + "q_proj.weight"]).view(t, 3, 16) * f
    k = pl.linear(h, w[p + "k_proj.weight"]).view(t, 1, 16) * f
    v = pl.linear(h, w[p + "v_proj.weight"]).view(t, 1, 16)
    x = x + pl.linear(pl.attention(q, k, v, pos).reshape(t, 48), w[p + "o_proj.weight"])
    h = pl.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-5)
    x = x + pl.swiglu_mlp(h, *(w[f"model.layers.1.mlp.{n}_proj.weight"] for n in ("gate", "up", "down")))
    return pl.linear(pl.rms_norm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"])


def test_routed_feed_forward_and_another_position_encoding():
    from tiny_llm_b200.engine import StepEntry, make_runner
    from tiny_llm_b200.parts import DecoderModel, register_part
    from tiny_llm_b200.weights import load_state, random_state

    register_part("ffn", "routed_relu", RoutedFeedForward)
    register_part("position", "position_scale", PositionScale)
    model = DecoderModel(toy_spec())
    specs = model.weight_specs()
    assert "model.layers.0.moe.experts.up" in specs and "model.layers.1.mlp.gate_proj.weight" in specs
    assert not model.graph_safe      # the toy feed-forward computes with torch: its steps are not captured
    state = random_state(specs, 5, 0.2, torch.float32)
    model.load(load_state(specs, state, torch.float32, DEV))
    runner = make_runner(model, "float32", DEV, max_tokens=128, page_size=8, max_requests=2)
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 101, (37,), generator=g).tolist()
    b = torch.randint(0, 101, (12,), generator=g).tolist()
    ref_a, ref_b = plain_toy(state, a), plain_toy(state, b)
    runner.cache.add_request("a"), runner.cache.add_request("b")
    got_a, got_b = [], []
    plan = [((0, 9), (0, 2)), ((9, 10), (2, 3)), ((10, 30), (3, 4)), ((30, 31), (4, 12)), ((31, 37), None)]
    for ra, rb in plan:
        entries = [StepEntry("a", a[ra[0]:ra[1]], range(ra[1] - ra[0]))]
        if rb:
            entries.append(StepEntry("b", b[rb[0]:rb[1]], range(rb[1] - rb[0])))
        out = runner.step(entries).cpu()
        got_a.append(out[: ra[1] - ra[0]].clone())
        if rb:
            got_b.append(out[ra[1] - ra[0]:].clone())
    assert runner.graph_replays == 0
    assert float((torch.cat(got_a) - ref_a).abs().max()) < 2e-5 * max(1.0, float(ref_a.abs().max()))
    assert float((torch.cat(got_b) - ref_b).abs().max()) < 2e-5 * max(1.0, float(ref_b.abs().max()))
