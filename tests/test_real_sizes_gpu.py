"""Replay at the real layer sizes: the kernels and paths that serving and the benchmark run.

Three shapes, each with a few of the model's layers so that the plain implementation stays fast on the
CPU (layer sizes, heads, vocabulary and positions are the model's own):
  TinyLlama-1.1B  4 of 22 layers: hidden 2048, 32 heads over 4 key/value heads of 64, 5632, vocab 32000
  Llama-2-7B      2 of 32 layers: hidden 4096, 32 heads = 32 key/value heads of 128, 11008, vocab 32000
  Llama-3-8B      2 of 32 layers: hidden 4096, 32 heads over 8 key/value heads of 128, 14336,
                  vocab 128256, 8192 positions, theta 500000
A 2,048-token prompt runs whole, in portions of 512/300/2/..., and with its last 32 tokens one by one
(contexts 2,016 to 2,047: decode attention over many key slices, replayed CUDA graphs); at the
TinyLlama shape eight requests live at contexts above 1,000 with portions of newcomers beside their
decoded tokens and so few pages that they are used again.  Logits are compared at chosen places (the
first tokens, page and portion edges, the last 32) with the plain implementation.  bfloat16 is held to
the rounding yardstick of replay_util.  The 32-bit path is compared with the plain implementation run in
64-bit and held to 1e-4, or to four times the error that the plain implementation's own 32-bit run has
against its 64-bit run where that is larger: with attention as peaked as here the 32-bit plain run is
itself up to 1.4e-4 away from the 64-bit one, and the engine, which sums every product in ascending k
where the CPU library sums in blocks, was measured at 2.2 to 2.5 times the plain run's error at three
degrees of sharpening.  Between the cuts the 32-bit logits are equal bit for bit.

The query and key projections are scaled up so that attention is peaked: a wrong or missing key then
moves the logits far beyond rounding (with N(0, 0.02) alone attention over 2,000 keys is nearly flat
and a wrong page could hide); one test puts a wrong page into the cache on purpose (another page's keys
and values in every layer, as a wrong block-table entry would give) and checks that both comparisons
see it."""
import pytest
import torch

import plain_llama as pl
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BASE = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", rms_norm_eps=1e-5,
            tie_word_embeddings=False, initializer_range=0.02, torch_dtype="float32")
SHAPES = {
    "tinyllama": (dict(BASE, num_hidden_layers=4, hidden_size=2048, num_attention_heads=32, num_key_value_heads=4,
                       intermediate_size=5632, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=2048), 22, 2),
    "llama2_7b": (dict(BASE, num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=32,
                       intermediate_size=11008, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096), 32, 3),
    "llama3_8b": (dict(BASE, num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                       intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192), 32, 4),
}
SHARPEN = 3.0      # factor on q_proj and k_proj: scores get a spread of several units instead of under one
PROMPT = 2048
TAIL = 32
WANT = sorted(set([0, 1, 2, 3, 15, 16, 17, 63, 64, 65, 127, 128, 129, 511, 512, 811, 812, 813, 814, 1023, 1024, 1324,
                   1325] + list(range(PROMPT - TAIL, PROMPT))))
PORTIONS = [512, 300, 2, 511, 1, 256, 129, 2, 64, 271]   # sums to 2,048


def make_state(cfg, seed):
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import random_state
    specs = DecoderModel(cfg.model_spec()).weight_specs()
    # drawn on the GPU (a billion normal numbers take a minute on the CPU), kept on the host for both sides
    state = {k: v.cpu() for k, v in random_state(specs, seed, cfg.initializer_range, torch.float32, device=DEV).items()}
    for name in state:
        if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            state[name] *= SHARPEN
    return specs, state


@pytest.fixture(scope="module", params=list(SHAPES))
def shape(request):
    """Configuration, weights, one 2,048-token request and the plain implementation's logits at WANT."""
    from tiny_llm_b200.config import LlamaConfig
    d, layers_of_model, seed = SHAPES[request.param]
    cfg = LlamaConfig.from_dict(d)
    specs, state = make_state(cfg, seed)
    toks = ru.make_requests(cfg.vocab_size, [PROMPT], seed)["r0"]
    pcfg = cfg.to_dict()
    ref64 = pl.forward(pcfg, state, toks, rows=WANT, dtype=torch.float64).float()
    ref32 = pl.forward(pcfg, state, toks, rows=WANT)
    wq = {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in state.items()}
    ref16 = pl.forward(pcfg, wq, toks, quant=pl.bf16_quant, rows=WANT)
    del wq
    return dict(name=f"{request.param} ({cfg.num_hidden_layers} of {layers_of_model} layers)", cfg=cfg, specs=specs,
                state=state, toks=toks, ref64=ref64, ref32=ref32, ref16=ref16, tol32=tolerance32(ref32, ref64))


def tolerance32(ref32, ref64):
    """1e-4, or four times the plain implementation's own 32-bit error where that is larger."""
    return max(1e-4, 4.0 * float((ref32 - ref64).abs().max()))


def build_runner(cfg, specs, state, dtype, max_tokens, max_requests=8, max_step=2048):
    from tiny_llm_b200.cache import CacheManager
    from tiny_llm_b200.engine import ModelRunner, parse_dtype
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state
    model = DecoderModel(cfg.model_spec())
    model.load(load_state(specs, state, parse_dtype(dtype), DEV))
    cache = CacheManager(model.cache_needs(), max_tokens=max_tokens, page_size=16, max_slots=max_requests)
    cache.allocate_storage(parse_dtype(dtype), DEV)
    for g in cache.groups:
        g.kv.fill_(float("nan"))
    return ModelRunner(model, cache, parse_dtype(dtype), DEV, max_tokens_per_step=max_step,
                       max_requests_per_step=max_requests)


def cut(toks, sizes, rid, want=WANT):
    """One request cut into steps of the given sizes; logits are asked for at the places of `want`."""
    steps, lo = [], 0
    for i, n in enumerate(sizes):
        hi = lo + n
        steps.append({"entries": [{"id": rid, "tokens": toks[lo:hi], "want": [p - lo for p in want if lo <= p < hi]}],
                      "end": [rid] if hi == len(toks) else []})
        lo = hi
    assert lo == len(toks)
    return steps


def three_cuts(runner, toks, vocab):
    whole = ru.run_trace_runner(runner, cut(toks, [PROMPT], "whole"), vocab)["whole"]
    portions = ru.run_trace_runner(runner, cut(toks, PORTIONS, "portions"), vocab)["portions"]
    replays = runner.graph_replays
    tail = ru.run_trace_runner(runner, cut(toks, [PROMPT - TAIL] + [1] * TAIL, "tail"), vocab)["tail"]
    assert runner.graph_replays - replays >= TAIL - 2, "the one-token steps did not replay a captured graph"
    return {"whole": whole, "portions": portions, "tail": tail}


def test_float32_at_real_sizes_matches_plain_and_cuts_agree_bitwise(shape):
    from tiny_llm_b200 import ops
    runner = build_runner(shape["cfg"], shape["specs"], shape["state"], "float32", max_tokens=PROMPT + 64)
    got = three_cuts(runner, shape["toks"], shape["cfg"].vocab_size)
    ops.check_status()
    worst = 0.0
    for how, g in got.items():
        assert g.shape == shape["ref64"].shape
        assert not torch.isnan(g).any(), how
        d = float((g - shape["ref64"]).abs().max())
        assert d <= shape["tol32"], (shape["name"], how, d, shape["tol32"])
        worst = max(worst, d)
    ru.record_margin(f"{shape['name']} whole/portions/tail (limit {shape['tol32']:.2e}, plain 32-bit run itself "
                     f"{float((shape['ref32'] - shape['ref64']).abs().max()):.2e})", "float32", worst, "|diff| to the 64-bit plain run")
    assert torch.equal(got["portions"], got["whole"]) and torch.equal(got["tail"], got["whole"])


def test_bfloat16_at_real_sizes_within_the_rounding_yardstick(shape):
    from tiny_llm_b200 import ops
    runner = build_runner(shape["cfg"], shape["specs"], shape["state"], "bfloat16", max_tokens=PROMPT + 64)
    got = three_cuts(runner, shape["toks"], shape["cfg"].vocab_size)
    ops.check_status()
    for how, g in got.items():
        assert not torch.isnan(g).any(), how
        ru.compare({"x" + "r": g}, {"r": shape["ref16"]}, "x", "bfloat16", f"{shape['name']} {how}", {"r": shape["ref32"]})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wrong_page_in_the_cache_is_seen_by_the_comparison(shape, dtype):
    """After the prompt, one page of the request (keys 1,120 to 1,135 of 2,016) is overwritten in every
    layer with another of its pages, keys and values, which is what a wrong block-table entry gives; the
    logits of the 32 tokens decoded after that must fall outside the tolerance.  (If they did not, the
    comparisons above could not tell a wrong page from rounding.)"""
    from tiny_llm_b200.engine import StepEntry
    cfg, toks = shape["cfg"], shape["toks"]
    runner = build_runner(cfg, shape["specs"], shape["state"], dtype, max_tokens=PROMPT + 64)
    head = PROMPT - TAIL
    runner.cache.add_request("x")
    runner.step([StepEntry("x", toks[:head], [])])
    table = runner.cache.block_table(0, "x")
    kv = runner.cache.groups[0].kv
    kv[:, :, table[70]] = kv[:, :, table[20]]
    rows = [runner.step([StepEntry("x", [toks[i]], [0])]).cpu().clone() for i in range(head, PROMPT)]
    runner.cache.free_request("x")
    got = torch.cat(rows)
    tail_rows = [WANT.index(p) for p in range(head, PROMPT)]
    if dtype == "float32":
        d = float((got - shape["ref64"][tail_rows]).abs().max())
        ru.record_margin(f"{shape['name']} with a wrong page", dtype, d / shape["tol32"], "|diff| / tolerance (must exceed 1)")
        assert d > shape["tol32"], (d, shape["tol32"])
    else:
        r16, r32 = shape["ref16"][tail_rows], shape["ref32"][tail_rows]
        ratio = float((got - r16).abs().max()) / float((r16 - r32).abs().max())
        ru.record_margin(f"{shape['name']} with a wrong page", dtype, ratio, "|diff| / tolerance (must exceed 1)")
        assert ratio > 1.0, ratio


# ----------------------------------------------------------------------------- eight live requests


def mixed_trace(reqs, max_live=8, portion=400, decode=40):
    """One request is admitted per step while fewer than max_live are live; a request runs its prompt
    in portions of `portion` tokens (the last one shorter), then its last `decode` tokens one by one.
    Logits are wanted for the decoded tokens and the one before them."""
    waiting = list(reqs.items())
    live, steps = {}, []
    while waiting or live:
        if waiting and len(live) < max_live:
            rid, t = waiting.pop(0)
            live[rid] = [t, 0]
        entries, end = [], []
        for rid in list(live):
            t, pos = live[rid]
            first_decoded = len(t) - decode
            n = 1 if pos >= first_decoded else min(portion, first_decoded - pos)
            want = [i for i in range(n) if pos + i >= first_decoded - 1]
            entries.append({"id": rid, "tokens": t[pos:pos + n], "want": want})
            live[rid][1] = pos + n
            if pos + n == len(t):
                end.append(rid)
                del live[rid]
        steps.append({"entries": entries, "end": end})
    return steps


CROWD_ROW0 = 960    # the plain implementation's logits are kept from this position on


@pytest.fixture(scope="module")
def crowd():
    """Twelve requests over four different token sequences (a request is a prefix of its sequence, so
    four runs of the plain implementation serve all twelve)."""
    from tiny_llm_b200.config import LlamaConfig
    d, _, seed = SHAPES["tinyllama"]
    cfg = LlamaConfig.from_dict(d)
    specs, state = make_state(cfg, seed)
    seqs = ru.make_requests(cfg.vocab_size, [1216] * 4, 77)
    lengths = [1216, 1100, 1040, 1201, 1185, 1111, 1216, 1024, 1090, 1150, 1216, 1057]
    reqs = {f"q{i}": seqs[f"r{i % 4}"][:n] for i, n in enumerate(lengths)}
    pcfg = cfg.to_dict()
    wq = {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in state.items()}
    rows = list(range(CROWD_ROW0, 1216))
    ref64 = {k: pl.forward(pcfg, state, t, rows=rows, dtype=torch.float64).float() for k, t in seqs.items()}
    ref32 = {k: pl.forward(pcfg, state, t, rows=rows) for k, t in seqs.items()}
    ref16 = {k: pl.forward(pcfg, wq, t, quant=pl.bf16_quant, rows=rows) for k, t in seqs.items()}
    return cfg, specs, state, reqs, lengths, ref64, ref32, ref16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eight_live_requests_beyond_1000_tokens_with_pages_used_again(crowd, dtype):
    cfg, specs, state, reqs, lengths, ref64, ref32, ref16 = crowd
    decode = 40
    steps = mixed_trace(reqs, decode=decode)
    need = ru.tokens_needed(steps)
    assert need < sum(-(-n // 64) * 64 for n in lengths)          # the pool cannot hold all twelve: pages come back
    runner = build_runner(cfg, specs, state, dtype, max_tokens=need, max_requests=8, max_step=2048)
    most_live = max(len(s["entries"]) for s in steps)
    decode_only = sum(1 for s in steps if len(s["entries"]) == 8 and all(len(e["tokens"]) == 1 for e in s["entries"]))
    assert most_live == 8 and decode_only > 10
    got = ru.run_trace_runner(runner, steps, cfg.vocab_size)
    assert runner.graph_replays > 0
    assert runner.cache.groups[0].pool.num_used == 0
    worst = 0.0
    for i, (rid, toks) in enumerate(reqs.items()):
        n = len(toks)
        rows = slice(n - decode - 1 - CROWD_ROW0, n - CROWD_ROW0)
        r32 = ref32[f"r{i % 4}"][rows]
        g = got[rid]
        assert g.shape == r32.shape and not torch.isnan(g).any(), rid
        if dtype == "float32":
            r64 = ref64[f"r{i % 4}"][rows]
            tol = tolerance32(r32, r64)
            d = float((g - r64).abs().max())
            assert d <= tol, (rid, d, tol)
            worst = max(worst, d / tol)
        else:
            r16 = ref16[f"r{i % 4}"][rows]
            tol = float((r16 - r32).abs().max())
            d = float((g - r16).abs().max())
            assert d <= tol, (rid, d, tol)
            worst = max(worst, d / tol)
    ru.record_margin("tinyllama (4 of 22 layers) eight live requests, pages used again", dtype, worst,
                     "|diff| / tolerance")
