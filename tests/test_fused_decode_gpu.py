"""The decode step as one persistent kernel (an option of the runner) against the plain
implementation: the last 32 tokens one by one, and mixed batches whose decode-only steps carry up
to four requests, with so few pages that they are used again."""
import pytest

import replay_util as ru
from conftest import TINY
from test_replay_gpu import LENGTHS, runner_for

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cases(model_dirs):
    out = {}
    for name, (cfg, page, seed) in TINY.items():
        reqs = ru.make_requests(cfg["vocab_size"], LENGTHS[name], seed + 10)
        out[name] = (model_dirs[name], cfg, page, reqs,
                     {d: ru.plain_logits(model_dirs[name], reqs, d) for d in ("float32", "bfloat16")})
    return out


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("how", ["tail", "mixed"])
def test_fused_decode_step(cases, name, how, monkeypatch):
    monkeypatch.setenv("TLLM_FUSED_DECODE", "1")
    model_dir, cfg, page, reqs, ref = cases[name]
    steps, prefix = {"tail": (ru.trace_tail(reqs), "t"), "mixed": (ru.trace_mixed(reqs, 4), "m")}[how]
    runner = runner_for(model_dir, "bfloat16", page, ru.tokens_needed(steps, round_to=page))
    got = ru.run_trace_runner(runner, steps, cfg["vocab_size"])
    assert runner._fused is not None and runner.fused_steps > 0, "the fused kernel did not take the decode steps"
    ru.compare(got, ref["bfloat16"], prefix, "bfloat16", f"fused decode, {how}", ref["float32"])
    from tiny_llm_b200 import ops
    ops.check_status()
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def test_fused_decode_is_refused_where_it_does_not_fit(cases, monkeypatch):
    """32-bit, or a layer that reads another layer's cache: the runner keeps the part-by-part path."""
    monkeypatch.setenv("TLLM_FUSED_DECODE", "1")
    from tiny_llm_b200.engine.fused_decode import FusedDecode
    model_dir, cfg, page, reqs, ref = cases["A"]
    runner = runner_for(model_dir, "float32", page, 256)
    assert FusedDecode.build(runner) is None
