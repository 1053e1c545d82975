"""Replay on the GPU against the plain implementation, in 32-bit and in bfloat16: whole; most in one
step and the last 32 tokens one by one; portions of changing size; mixed with few pages."""
import pytest
import torch

import replay_util as ru
from conftest import TINY

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [100, 64, 33, 47, 128, 17, 80, 51], "B": [97, 2, 40, 255, 33, 64, 13, 150], "C": [70, 192, 35, 49]}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def cases(model_dirs):
    out = {}
    for name, (cfg, page, seed) in TINY.items():
        reqs = ru.make_requests(cfg["vocab_size"], LENGTHS[name], seed + 10)
        out[name] = (model_dirs[name], cfg, page, reqs, {d: ru.plain_logits(model_dirs[name], reqs, d) for d in DTYPES})
    return out


def runner_for(model_dir, dtype, page, max_tokens, poison=True):
    from tiny_llm_b200.engine import load_model, make_runner
    _, model = load_model(model_dir, dtype, "cuda:0")
    runner = make_runner(model, dtype, "cuda:0", max_tokens=max_tokens, page_size=page, max_requests=8,
                         max_tokens_per_step=1024)
    if poison:  # a slot that is read before it is written shows as NaN in the logits
        for g in runner.cache.groups:
            g.kv.fill_(float("nan"))
    return runner


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_program(cases, name, dtype):
    """All four ways of cutting, through bin/trace_run as a user runs it, with the smallest pool."""
    model_dir, cfg, page, reqs, ref = cases[name]
    some = dict(list(reqs.items())[:5])
    steps = (ru.trace_whole(some) + ru.trace_tail(some) + ru.trace_portions(some, 1) + ru.trace_mixed(reqs, 2))
    got = ru.run_trace_cli(model_dir, dtype, steps, cfg["vocab_size"])
    ref_some = {k: ref[dtype][k] for k in some}
    f32 = ref["float32"]
    ru.compare(got, ref_some, "w", dtype, "whole", f32)
    ru.compare(got, ref_some, "t", dtype, "last 32 one by one", f32)
    ru.compare(got, ref_some, "p", dtype, "portions", f32)
    ru.compare(got, ref[dtype], "m", dtype, "mixed", f32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_replay_in_process(cases, name, dtype, how):
    model_dir, cfg, page, reqs, ref = cases[name]
    steps, prefix = {"whole": (ru.trace_whole(reqs), "w"), "tail": (ru.trace_tail(reqs), "t"),
                     "portions": (ru.trace_portions(reqs, 3), "p"), "mixed": (ru.trace_mixed(reqs, 4), "m")}[how]
    runner = runner_for(model_dir, dtype, page, ru.tokens_needed(steps, round_to=page))
    got = ru.run_trace_runner(runner, steps, cfg["vocab_size"])
    ru.compare(got, ref[dtype], prefix, dtype, how, ref["float32"])
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)
    if how == "mixed":   # so few pages that they were used again
        total = sum(-(-len(t) // page) for t in reqs.values())
        assert total > runner.cache.groups[0].pool.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_twice_with_different_pages_gives_the_same_logits(cases, name, dtype):
    """The same trace with another page size and a larger pool: beyond rounding nothing moves."""
    model_dir, cfg, page, reqs, ref = cases[name]
    steps = ru.trace_mixed(reqs, 7)
    a = ru.run_trace_runner(runner_for(model_dir, dtype, page, ru.tokens_needed(steps, page)), steps, cfg["vocab_size"])
    b = ru.run_trace_runner(runner_for(model_dir, dtype, 4 * page, 4096), steps, cfg["vocab_size"])
    for rid in a:
        tol = 1e-6 if dtype == "float32" else ru.tolerance(ref[dtype][rid[1:]], dtype, ref["float32"][rid[1:]])
        assert float((a[rid] - b[rid]).abs().max()) <= tol, rid
    if dtype == "float32":   # the 32-bit path orders its sums by position only: cuts do not move a bit
        whole = ru.run_trace_runner(runner_for(model_dir, dtype, page, 4096), ru.trace_whole(reqs), cfg["vocab_size"])
        for rid in reqs:
            assert torch.equal(whole["w" + rid], a["m" + rid]), rid


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_and_first_tokens(cases, name, dtype):
    model_dir, cfg, page, _, _ = cases[name]
    n = cfg["max_position_embeddings"]
    reqs = ru.make_requests(cfg["vocab_size"], [n, 1, 2, 3], 99)
    ref = ru.plain_logits(model_dir, reqs, dtype)
    ref32 = ref if dtype == "float32" else ru.plain_logits(model_dir, reqs, "float32")
    # r0: one prompt token, then every further token one by one up to the model's last position
    steps = ru.trace_tail({"r0": reqs["r0"]}, tail=n - 1) + ru.trace_whole({k: reqs[k] for k in ("r1", "r2", "r3")})
    runner = runner_for(model_dir, dtype, page, ru.tokens_needed(steps, page))
    got = ru.run_trace_runner(runner, steps, cfg["vocab_size"])
    ru.compare(got, {"r0": ref["r0"]}, "t", dtype, "long decoding", ref32)
    ru.compare(got, {k: ref[k] for k in ("r1", "r2", "r3")}, "w", dtype, "first tokens", ref32)
    with pytest.raises(ValueError, match="limit"):
        runner.cache.add_request("x")
        from tiny_llm_b200.engine import StepEntry
        runner.step([StepEntry("x", [1] * (n + 1), [])])


def test_step_refuses_what_it_cannot_hold(cases):
    from tiny_llm_b200.engine import OutOfPages, StepEntry
    model_dir, cfg, page, _, _ = cases["A"]
    runner = runner_for(model_dir, "float32", page, 32)
    runner.cache.add_request("a"), runner.cache.add_request("b")
    runner.step([StepEntry("a", [1] * 20, [])])
    free = runner.cache.groups[0].pool.num_free
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", [1], []), StepEntry("b", [1] * 17, [0])])
    assert runner.cache.groups[0].pool.num_free == free      # nothing was taken
    with pytest.raises(ValueError, match="token id"):
        runner.step([StepEntry("b", [cfg["vocab_size"]], [0])])
    with pytest.raises(KeyError):
        runner.step([StepEntry("nobody", [1], [0])])


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_id_that_lives_twice_decodes_from_its_new_pages(cases, dtype):
    """Steps in which every request brings one token take their block tables from rows kept per request
    id.  An id that ends and comes back holds other pages: its kept row must not survive it."""
    from tiny_llm_b200.engine import StepEntry
    model_dir, cfg, page, _, _ = cases["A"]
    reqs = ru.make_requests(cfg["vocab_size"], [40, 50, 21], 123)       # first life of x, second life of x, y
    names = {"x1": reqs["r0"], "x2": reqs["r1"], "y": reqs["r2"]}
    ref = ru.plain_logits(model_dir, names, dtype)
    ref32 = ref if dtype == "float32" else ru.plain_logits(model_dir, names, "float32")
    runner = runner_for(model_dir, dtype, page, 192)
    cache = runner.cache

    def live(rid, toks, tail, beside=None):
        """The request's prompt in one step, its last `tail` tokens one by one (alone, or beside `beside`)."""
        cache.add_request(rid)
        head = len(toks) - tail
        rows = [runner.step([StepEntry(rid, toks[:head], range(head))]).cpu().clone()]
        for i in range(head, len(toks)):
            entries = [StepEntry(rid, [toks[i]], [0])]
            if beside is not None:
                entries.append(StepEntry(beside[0], [beside[1].pop(0)], [0]))
            rows.append(runner.step(entries).cpu()[:1].clone())
        return torch.cat(rows), list(cache.block_table(0, rid))

    got1, pages1 = live("x", names["x1"], 10)
    cache.free_request("x")
    cache.add_request("y")                                   # y takes the pages x gave back
    runner.step([StepEntry("y", names["y"][:12], [])])
    y_rest = list(names["y"][12:])
    got2, pages2 = live("x", names["x2"], 9, beside=("y", y_rest))   # x again, other pages, decoding beside y
    assert pages1[: len(pages2)] != pages2[: len(pages1)] and set(pages2).isdisjoint(cache.block_table(0, "y"))
    assert runner.graph_replays > 0
    cache.free_request("x"), cache.free_request("y")
    ru.compare({"ax1": got1, "ax2": got2}, {"x1": ref["x1"], "x2": ref["x2"]}, "a", dtype, "a request id that lives twice",
               {"x1": ref32["x1"], "x2": ref32["x2"]})


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_a_graph_bucket_of_the_context(tmp_path_factory, dtype):
    """Replayed graphs are keyed by the power-of-two bucket of the longest context (256, 512, ...): a request
    decodes from 247 to 275 tokens, across the edge, beside a short one (whose key slices are empty in the
    larger bucket)."""
    from conftest import TINY_A
    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.weights import write_random_model
    cfg = dict(TINY_A, max_position_embeddings=1024)
    d = str(tmp_path_factory.mktemp("tiny_long"))
    write_random_model(d, LlamaConfig.from_dict(cfg), seed=7, dtype=torch.float32)
    reqs = ru.make_requests(cfg["vocab_size"], [275, 40], 5)
    ref = ru.plain_logits(d, reqs, dtype)
    ref32 = ref if dtype == "float32" else ru.plain_logits(d, reqs, "float32")
    long_t, short_t = reqs["r0"], reqs["r1"]
    steps = [{"entries": [{"id": "gr0", "tokens": long_t[:247], "want": list(range(247))},
                          {"id": "gr1", "tokens": short_t[:12], "want": list(range(12))}], "end": []}]
    for i in range(28):
        steps.append({"entries": [{"id": "gr0", "tokens": [long_t[247 + i]], "want": [0]},
                                  {"id": "gr1", "tokens": [short_t[12 + i]], "want": [0]}],
                      "end": ["gr0", "gr1"] if i == 27 else []})
    runner = runner_for(d, dtype, 16, 384)
    got = ru.run_trace_runner(runner, steps, cfg["vocab_size"])
    assert runner.graph_replays >= 20 and len(runner._graphs) == 2       # one graph per bucket, both replayed
    ru.compare(got, ref, "g", dtype, "decoding across a graph bucket", ref32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_steps_run_again_from_the_tape_of_their_launches(cases, name, dtype):
    """A step whose sizes (tokens, requests, wanted places, longest portion, context bucket) were seen before is not
    walked through the model's Python code again: the launches noted the first time run again, and the kernels read
    the new ids, positions, tables and slots from device memory.  Two rounds of the same shapes with other contents
    (other ids, other request ids, other pages since the pool is used again) on a runner with tapes and on one
    without: in 32-bit the logits agree to the bit, in bfloat16 within what atomic sums allow, and both match plain."""
    from tiny_llm_b200.engine import StepEntry
    model_dir, cfg, page, reqs, ref = cases[name]
    lens = [37, 5, 64, 18]
    rounds = [ru.make_requests(cfg["vocab_size"], lens, 500 + r) for r in range(3)]
    outs = {}
    for taped in (True, False):
        runner = runner_for(model_dir, dtype, page, 4 * 128)
        runner.use_tapes = taped
        got = []
        for r, rq in enumerate(rounds):
            ids = list(rq)
            toks = [rq[i] for i in ids]
            live = [f"{r}-{i}" for i in ids]
            for rid in live:
                runner.cache.add_request(rid)
            # a portion of each beside single tokens of others, cut so that the shapes repeat from round to round
            steps = [[(0, 0, 20, [19]), (1, 0, 3, [])],
                     [(0, 20, 37, [16]), (1, 3, 4, [0]), (2, 0, 40, [])],
                     [(1, 4, 5, [0]), (2, 40, 64, [23]), (3, 0, 18, [0, 17])]]
            for step in steps:
                entries = [StepEntry(live[q], toks[q][a:b], want) for q, a, b, want in step]
                logits = runner.step(entries)
                got.append(logits.float().cpu().clone())
            for rid in live:
                runner.cache.free_request(rid)
        outs[taped] = (got, runner.tape_replays)
    assert outs[True][1] >= 6 and outs[False][1] == 0        # rounds two and three ran from the tapes of round one
    for a, b in zip(outs[True][0], outs[False][0]):
        if dtype == "float32":
            assert torch.equal(a, b)
        else:
            assert float((a - b).abs().max()) <= 1e-2 * max(1.0, float(b.abs().max()))
    # and against the plain implementation: the last place of request 0 of every round
    import plain_llama as pl
    c, w = pl.load_config(model_dir), pl.load_weights(model_dir)
    for r, rq in enumerate(rounds):
        t0 = rq[list(rq)[0]]
        want = pl.forward(c, w, t0, dtype=torch.float32)[36]
        have = outs[True][0][3 * r + 1][0]
        tol = 2e-5 if dtype == "float32" else 0.05
        assert float((have - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
