"""Each part alone on the GPU, built from a spec through the registry, against the plain functions."""
import math
import types

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def context(dtype, positions=None, token_request=None):
    """A step context for one request whose tokens are at `positions`."""
    from tiny_llm_b200.engine import Workspace
    batch = types.SimpleNamespace(
        positions=None if positions is None else positions.to(torch.int32).to(DEV),
        token_request=None if token_request is None else token_request.to(torch.int32).to(DEV))
    if positions is not None:
        n, first = len(positions), int(positions[0])
        batch.cu_q = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        batch.q_start = torch.tensor([first], dtype=torch.int32, device=DEV)
        batch.num_requests, batch.max_q_len, batch.max_kv_len = 1, n, first + n
    return types.SimpleNamespace(dtype=DT[dtype], device=torch.device(DEV), workspace=Workspace(DEV), batch=batch)


def tol(dtype, ref):
    return (2e-5 if dtype == "float32" else 2.0 ** -6) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", DT)
def test_norm_part(dtype):
    from tiny_llm_b200.config import PartSpec
    from tiny_llm_b200.parts import build_part
    torch.manual_seed(0)
    part = build_part("norm", PartSpec("rms_norm", {"size": 208, "eps": 3e-4}))
    assert [(s.name, s.shape) for s in part.weight_specs("x.norm")] == [("x.norm.weight", (208,))]
    w = torch.randn(208)
    part.load("x.norm", {"x.norm.weight": w.to(DEV)})
    x = torch.randn(11, 208)
    got = part.forward(context(dtype), x.to(DEV)).float().cpu()
    ref = pl.rms_norm(x, w, 3e-4)
    assert float((got - ref).abs().max()) <= tol(dtype, ref)


def test_rotary_part_tables():
    from tiny_llm_b200.config import PartSpec
    from tiny_llm_b200.parts import build_part
    part = build_part("position", PartSpec("rotary", {"head_dim": 48, "theta": 12345.0, "max_positions": 300}))
    part.prepare(DEV)
    cos, sin = pl.rope_tables(300, 48, 12345.0)
    assert torch.equal(part.cos.cpu(), cos) and torch.equal(part.sin.cpu(), sin) and part.rot_dim == 48


@pytest.mark.parametrize("dtype", DT)
def test_feed_forward_part(dtype):
    from tiny_llm_b200.config import PartSpec
    from tiny_llm_b200.parts import build_part
    torch.manual_seed(1)
    h, i = 80, 208
    part = build_part("ffn", PartSpec("swiglu", {"hidden_size": h, "intermediate_size": i}))
    names = [s.name for s in part.weight_specs("m.")]
    assert names == ["m.gate_proj.weight", "m.up_proj.weight", "m.down_proj.weight"]
    w = {"m.gate_proj.weight": torch.randn(i, h) * 0.2, "m.up_proj.weight": torch.randn(i, h) * 0.2,
         "m.down_proj.weight": torch.randn(h, i) * 0.2}
    wq = {k: v.to(DT[dtype]) for k, v in w.items()}
    part.load("m.", {k: v.to(DEV) for k, v in wq.items()})
    y = torch.randn(13, h).to(DT[dtype])
    resid = torch.full((13, h), 0.25, device=DEV)
    part.forward(context(dtype), y.to(DEV), resid)
    quant = pl.no_quant if dtype == "float32" else pl.bf16_quant
    ref = pl.swiglu_mlp(y.float(), *(wq[n].float() for n in names), quant=quant)
    assert float((resid.cpu() - 0.25 - ref).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_over_two_steps(dtype, window):
    """The mixer alone: a portion of 20 tokens, then 5 more, through its own pages."""
    from tiny_llm_b200.config import PartSpec
    from tiny_llm_b200.engine import KVView
    from tiny_llm_b200.parts import build_part
    torch.manual_seed(2)
    hid, nq, nkv, hd, page = 80, 6, 3, 32, 8
    rope = PartSpec("rotary", {"head_dim": hd, "theta": 777.0, "max_positions": 64})
    part = build_part("mixer", PartSpec("gqa_attention", {"hidden_size": hid, "num_heads": nq, "num_kv_heads": nkv,
                                                           "head_dim": hd, "position": rope, "window": window}))
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (nkv, hd, window)
    w = {"a.q_proj.weight": torch.randn(nq * hd, hid) * 0.3, "a.k_proj.weight": torch.randn(nkv * hd, hid) * 0.3,
         "a.v_proj.weight": torch.randn(nkv * hd, hid) * 0.3, "a.o_proj.weight": torch.randn(hid, nq * hd) * 0.3}
    assert sorted(s.name for s in part.weight_specs("a.")) == sorted(w)
    wq = {k: v.to(DT[dtype]) for k, v in w.items()}
    part.load("a.", {k: v.to(DEV) for k, v in wq.items()})
    x = torch.randn(25, hid).to(DT[dtype])
    kv = torch.full((2, 6, nkv, page, hd), float("nan"), dtype=DT[dtype], device=DEV)
    pages = [4, 1, 5, 0]
    table = torch.tensor([pages + [-1]], dtype=torch.int32, device=DEV)
    outs = []
    for lo, hi in ((0, 20), (20, 25)):
        pos = torch.arange(lo, hi)
        slots = torch.tensor([pages[p // page] * page + p % page for p in range(lo, hi)], dtype=torch.int32, device=DEV)
        ctx = context(dtype, pos, torch.zeros(hi - lo))
        resid = torch.zeros(hi - lo, hid, device=DEV)
        part.forward(ctx, x[lo:hi].to(DEV), resid, KVView(kv[0], kv[1], table, slots, page))
        outs.append(resid.cpu())
    got = torch.cat(outs)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": hid}
    cos, sin = pl.rope_tables(64, hd, 777.0)
    quant = pl.no_quant if dtype == "float32" else pl.bf16_quant
    ref = pl.attention_block(x.float(), {k: v.float() for k, v in wq.items()}, "a.", cfg, cos, sin, torch.arange(25),
                             quant=quant, window=window)
    assert float((got - ref).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DT)
def test_run_order_names_a_layer_twice_and_shares_a_cache(dtype):
    """Order [0, 1, 1, 2->reads call 0's cache]: layer 1 runs twice with a cache per call; the last
    call has no keys of its own and attends over the first call's."""
    import dataclasses
    from conftest import TINY_A
    from tiny_llm_b200.cache import CacheManager
    from tiny_llm_b200.config import LayerCall, LlamaConfig
    from tiny_llm_b200.engine import ModelRunner, StepEntry
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state, random_state
    cfg = LlamaConfig.from_dict(dict(TINY_A, num_hidden_layers=3))
    spec = cfg.model_spec()
    spec = dataclasses.replace(spec, order=[LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(2, reads_cache_of=0)])
    model = DecoderModel(spec)
    specs = model.weight_specs()
    assert "model.layers.2.self_attn.k_proj.weight" not in specs and "model.layers.2.self_attn.q_proj.weight" in specs
    assert [n is not None for n in model.cache_needs()] == [True, True, True, False]
    state = random_state(specs, 4, 0.15, torch.float32)
    model.load(load_state(specs, state, DT[dtype], DEV))
    cache = CacheManager(model.cache_needs(), max_tokens=64, page_size=16, max_slots=2)
    assert cache.groups[0].num_entries == 3
    cache.allocate_storage(DT[dtype], DEV)
    runner = ModelRunner(model, cache, DT[dtype], DEV, max_tokens_per_step=64, max_requests_per_step=2)
    toks = torch.randint(0, 256, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    cache.add_request("a")
    parts = [runner.step([StepEntry("a", toks[:23], range(23))]).cpu().clone(),
             runner.step([StepEntry("a", toks[23:], range(17))]).cpu().clone()]
    got = torch.cat(parts)
    # plain: the same order by hand
    wq = {k: (v if v.dim() == 1 or dtype == "float32" else v.to(torch.bfloat16).float()) for k, v in state.items()}
    quant = pl.no_quant if dtype == "float32" else pl.bf16_quant
    c = cfg.to_dict()
    cos, sin = pl.rope_tables(c["max_position_embeddings"], 16, c["rope_theta"])
    pos = torch.arange(40)
    x = pl.embedding(wq["model.embed_tokens.weight"], torch.tensor(toks))
    first_kv = None
    for call, layer in enumerate([0, 1, 1, 2]):
        p = f"model.layers.{layer}."
        h = quant(pl.rms_norm(x, wq[p + "input_layernorm.weight"], c["rms_norm_eps"]))
        q = quant(pl.apply_rope(quant(pl.linear(h, wq[p + "self_attn.q_proj.weight"])).view(40, 4, 16), cos, sin, pos))
        if layer != 2:
            k = quant(pl.apply_rope(quant(pl.linear(h, wq[p + "self_attn.k_proj.weight"])).view(40, 2, 16), cos, sin, pos))
            v = quant(pl.linear(h, wq[p + "self_attn.v_proj.weight"])).view(40, 2, 16)
            if call == 0:
                first_kv = (k, v)
        else:
            k, v = first_kv
        o = quant(pl.attention(q, k, v, pos, quant=quant)).reshape(40, 64)
        x = x + pl.linear(o, wq[p + "self_attn.o_proj.weight"])
        h = quant(pl.rms_norm(x, wq[p + "post_attention_layernorm.weight"], c["rms_norm_eps"]))
        x = x + pl.swiglu_mlp(h, wq[p + "mlp.gate_proj.weight"], wq[p + "mlp.up_proj.weight"],
                              wq[p + "mlp.down_proj.weight"], quant)
    ref = pl.linear(quant(pl.rms_norm(x, wq["model.norm.weight"], c["rms_norm_eps"])), wq["lm_head.weight"])
    assert float((got - ref).abs().max()) <= tol(dtype, ref)
