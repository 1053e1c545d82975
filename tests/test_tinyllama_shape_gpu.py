"""The TinyLlama-1.1B layer sizes with random weights (seed 2, N(0, 0.02)): the 32-bit path must
match the plain implementation to 1e-4 for every way of cutting the work, and the cuts must agree
with each other bit for bit; the bfloat16 path is held to the rounding yardstick of replay_util."""
import pytest
import torch

import plain_llama as pl
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHAPE = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=22, hidden_size=2048,
             num_attention_heads=32, num_key_value_heads=4, intermediate_size=5632, vocab_size=32000,
             rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=2048, tie_word_embeddings=False,
             hidden_act="silu", initializer_range=0.02, torch_dtype="float32")


@pytest.fixture(scope="module")
def big():
    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import random_state
    cfg = LlamaConfig.from_dict(SHAPE)
    specs = DecoderModel(cfg.model_spec()).weight_specs()
    state = random_state(specs, 2, 0.02, torch.float32)
    reqs = ru.make_requests(32000, [72, 41], 5)
    pcfg = cfg.to_dict()
    ref32 = {rid: pl.forward(pcfg, state, toks) for rid, toks in reqs.items()}
    return cfg, specs, state, reqs, pcfg, ref32


def build_runner(cfg, specs, state, dtype):
    from tiny_llm_b200.engine import ModelRunner, parse_dtype
    from tiny_llm_b200.cache import CacheManager
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state
    model = DecoderModel(cfg.model_spec())
    model.load(load_state(specs, state, parse_dtype(dtype), DEV))
    cache = CacheManager(model.cache_needs(), max_tokens=160, page_size=16, max_slots=4)
    cache.allocate_storage(parse_dtype(dtype), DEV)
    for g in cache.groups:
        g.kv.fill_(float("nan"))
    return ModelRunner(model, cache, parse_dtype(dtype), DEV, max_tokens_per_step=256, max_requests_per_step=4)


def test_float32_matches_plain_and_cuts_agree_bitwise(big):
    cfg, specs, state, reqs, pcfg, ref32 = big
    runner = build_runner(cfg, specs, state, "float32")
    whole = ru.run_trace_runner(runner, ru.trace_whole(reqs), 32000)
    for rid, r in ref32.items():
        d = float((whole["w" + rid] - r).abs().max())
        assert d <= 1e-4, (rid, d)
    print(f"[margin] 1.1B shape float32: max |diff| = {max(float((whole['w' + k] - v).abs().max()) for k, v in ref32.items()):.2e}")
    tail = ru.run_trace_runner(runner, ru.trace_tail(reqs, tail=6), 32000)
    mixed = ru.run_trace_runner(runner, ru.trace_mixed(reqs, 3), 32000)
    portions = ru.run_trace_runner(runner, ru.trace_portions(reqs, 2), 32000)
    for rid in reqs:
        assert torch.equal(tail["t" + rid], whole["w" + rid]), rid
        assert torch.equal(mixed["m" + rid], whole["w" + rid]), rid
        assert torch.equal(portions["p" + rid], whole["w" + rid]), rid


def test_bfloat16_within_the_rounding_yardstick(big):
    cfg, specs, state, reqs, pcfg, ref32 = big
    wq = {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in state.items()}
    ref16 = {rid: pl.forward(pcfg, wq, toks, quant=pl.bf16_quant) for rid, toks in reqs.items()}
    runner = build_runner(cfg, specs, state, "bfloat16")
    got = ru.run_trace_runner(runner, ru.trace_whole(reqs) + ru.trace_mixed(reqs, 3) + ru.trace_tail(reqs, tail=6), 32000)
    ru.compare(got, ref16, "w", "bfloat16", "1.1B shape whole", ref32)
    ru.compare(got, ref16, "m", "bfloat16", "1.1B shape mixed", ref32)
    ru.compare(got, ref16, "t", "bfloat16", "1.1B shape tail", ref32)
    from tiny_llm_b200 import ops
    ops.check_status()
