"""Generation through the Python entry point and the command line, against the plain implementation."""
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as pl
from conftest import TINY

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_model(model_dir, dtype):
    cfg, w = pl.load_config(model_dir), pl.load_weights(model_dir)
    if dtype == "bfloat16":
        w = {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in w.items()}
    return cfg, w, (pl.no_quant if dtype == "float32" else pl.bf16_quant)


def check_greedy(cfg, w, quant, dtype, prompt, generated):
    """Every generated token is the plain implementation's first maximum given the tokens before it,
    or ties with it within the path's rounding."""
    seq = list(prompt)
    for tok in generated:
        logits = pl.forward(cfg, w, seq, quant=quant)[-1]
        best = pl.greedy(logits)
        slack = 2e-5 if dtype == "float32" else 2.0 ** -6 * float(logits.abs().max())
        assert float(logits[best] - logits[tok]) <= slack, (seq, tok, best)
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    from tiny_llm_b200 import Pipeline
    cfg_d, page, _ = TINY[name]
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(8, cfg_d["vocab_size"], (n,), generator=g).tolist() for n in (1, 7, 16, 33)]
    pipe = Pipeline(model_dirs[name], dtype=dtype, device=0, page_size=page, max_tokens=512, max_requests=4,
                    max_tokens_per_step=24, chunk=5)
    out = pipe.apply(prompts, max_new_tokens=16, do_sample=False, ignore_eos=True)
    assert [len(o) for o in out] == [16] * 4
    assert pipe.counters["chained"] > 0 and pipe.runner.graph_replays > 0   # decode steps ran ahead of the host, as graphs
    cfg, w, quant = plain_model(model_dirs[name], dtype)
    for p, o in zip(prompts, out):
        check_greedy(cfg, w, quant, dtype, p, o)
    assert pipe.runner.cache.groups[0].pool.num_used == 0
    # the same prompts one at a time give the same tokens in 32-bit (no dependence on the batch)
    if dtype == "float32":
        for p, o in zip(prompts, out):
            assert pipe.apply([p], max_new_tokens=16, do_sample=False, ignore_eos=True)[0] == o


def test_pushed_out_requests_are_recomputed_to_the_same_tokens(model_dirs):
    from tiny_llm_b200 import Pipeline
    cfg_d, page, _ = TINY["A"]
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(8, 256, (n,), generator=g).tolist() for n in (30, 25, 40, 12)]
    roomy = Pipeline(model_dirs["A"], dtype="float32", page_size=16, max_tokens=1024, max_requests=4)
    want = roomy.apply(prompts, max_new_tokens=40, do_sample=False, ignore_eos=True)
    tight = Pipeline(model_dirs["A"], dtype="float32", page_size=16, max_tokens=160, max_requests=4)
    got = tight.apply(prompts, max_new_tokens=40, do_sample=False, ignore_eos=True)
    assert tight.scheduler.counters["pushed_out"] > 0 and roomy.scheduler.counters["pushed_out"] == 0
    assert got == want
    assert tight.runner.cache.groups[0].pool.num_used == 0 and tight.runner.cache.slots.num_free == 4


@pytest.mark.parametrize("name", ["A", "B"])
def test_temperature_sampling_is_seeded_and_follows_the_chain(model_dirs, name):
    from tiny_llm_b200 import Pipeline
    from tiny_llm_b200.sampling import uniform_from
    cfg_d, page, _ = TINY[name]
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(8, cfg_d["vocab_size"], (n,), generator=g).tolist() for n in (2, 13, 40)]
    pipe = Pipeline(model_dirs[name], dtype="float32", page_size=page, max_tokens=1024, max_requests=4)
    kw = dict(max_new_tokens=24, do_sample=True, temperature=0.8, top_k=20, top_p=0.9, ignore_eos=True)
    a = pipe.apply(prompts, seed=11, **kw)
    b = pipe.apply(list(reversed(prompts)), seed=11, **kw)
    c = pipe.apply(prompts, seed=12, **kw)
    assert a != c
    # request i draws from stream seed + i: the same prompt with the same stream gives the same tokens in another batch
    assert pipe.apply([prompts[1]], seed=12, **kw)[0] == a[1]
    assert b[1] == pipe.apply([prompts[1]], seed=12, **kw)[0]
    cfg, w, quant = plain_model(model_dirs[name], "float32")
    for i, (p, o) in enumerate(zip(prompts, a)):
        seq = list(p)
        for n, tok in enumerate(o):
            logits = pl.forward(cfg, w, seq, quant=quant)[-1]
            ids, pr = pl.sampling_distribution(logits, 0.8, 20, 0.9)
            want = pl.multinomial(ids, pr, uniform_from(11 + i, n))
            if tok != want:   # only a draw within rounding of a boundary may differ
                cdf = torch.cumsum(pr, 0)
                j = ids.tolist().index(tok)
                u = uniform_from(11 + i, n)
                assert (float(cdf[j - 1]) if j else 0.0) - 1e-4 <= u <= float(cdf[j]) + 1e-4
            seq.append(tok)


def test_eos_ends_a_request(model_dirs):
    """Wherever the end-of-sequence id falls, the last two places included: there the chained step that ran
    too far has already ended the request by length when the id is read."""
    from tiny_llm_b200 import Pipeline
    pipe = Pipeline(model_dirs["A"], dtype="float32", max_tokens=512, max_requests=2)
    free = pipe.apply([[9, 8, 7]], max_new_tokens=12, do_sample=False, ignore_eos=True)[0]
    assert pipe.counters["chained"] > 0
    for at in (4, 10, 11):
        pipe.scheduler.eos = {free[at]}
        cut = pipe.apply([[9, 8, 7]], max_new_tokens=12, do_sample=False)[0]
        assert cut == free[: free.index(free[at]) + 1], at
        assert pipe.runner.cache.groups[0].pool.num_used == 0


def test_command_line(model_dirs):
    cmd = [sys.executable, "-m", "tiny_llm_b200", f"--model_path={model_dirs['A']}", "--max_new_tokens", "5",
           "--nodo_sample", "--dtype=float32", "--page_mode"]
    res = subprocess.run(cmd, input="9 8 7\n\n3, 4\n5\n\n", capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert res.returncode == 0, res.stderr
    outs = [l for l in res.stdout.splitlines() if l and l[0].isdigit()]
    assert len(outs) == 2 and all(len(l.split()) <= 5 for l in outs)
    from tiny_llm_b200 import Pipeline
    pipe = Pipeline(model_dirs["A"], dtype="float32", max_tokens=512, max_requests=2)
    assert outs[0] == " ".join(map(str, pipe.apply([[9, 8, 7]], max_new_tokens=5, do_sample=False)[0]))
    bad = subprocess.run([sys.executable, "-m", "tiny_llm_b200"], capture_output=True, text=True, cwd=ROOT)
    assert bad.returncode == 1 and "model_path" in bad.stderr


def test_command_line_random_weights_and_a_batch_of_prompts(model_dirs, tmp_path):
    """--random_weights --config --seed makes the model that write_random_model makes; with
    --prompt_per_line the lines of a block run as one batch through the scheduler (portions of
    --chunk tokens under --max_tokens_per_step), with the tokens each prompt gives alone."""
    import json
    from conftest import TINY_A
    from tiny_llm_b200 import Pipeline
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY_A))
    cmd = [sys.executable, "-m", "tiny_llm_b200", "--random_weights", f"--config={cfg_path}", "--seed=0",
           "--max_new_tokens=6", "--nodo_sample", "--dtype=float32", "--prompt_per_line", "--max_requests=3",
           "--max_tokens_per_step=8", "--chunk=5", "--num_pages=12", "--page_size=16"]
    lines = ["9 8 7 6 5 4 3 10 11 12 13 14", "3, 4", "5 6 7 8 9 10 11"]
    res = subprocess.run(cmd, input="\n".join(lines) + "\n\n", capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert res.returncode == 0, res.stderr
    outs = [l for l in res.stdout.splitlines() if l and l[0].isdigit()]
    assert len(outs) == 3
    pipe = Pipeline(model_dirs["A"], dtype="float32", max_tokens=512, max_requests=2)   # seed 0: the same weights
    for line, out in zip(lines, outs):
        prompt = [int(t) for t in line.replace(",", " ").split()]
        assert out == " ".join(map(str, pipe.apply([prompt], max_new_tokens=6, do_sample=False)[0]))
    bad = subprocess.run([sys.executable, "-m", "tiny_llm_b200", "--random_weights"], capture_output=True, text=True, cwd=ROOT)
    assert bad.returncode == 1 and "--config" in bad.stderr


def test_many_requests_through_one_engine_give_what_each_gives_alone(model_dirs):
    """Two dozen requests of random lengths through one engine with a small token budget and a pool that cannot hold
    them all: steps of every mix (portions beside decoded tokens, requests pushed out and computed again), many of them
    with sizes seen before, so that graphs are replayed and launches run again from their tapes, with other contents and
    other pages each time.  In 32-bit every request must get exactly the tokens it gets alone on an engine that walks
    the model's code for every step."""
    from tiny_llm_b200 import Pipeline
    cfg_d, page, _ = TINY["B"]
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(1, 60, (24,), generator=g).tolist()
    news = torch.randint(4, 30, (24,), generator=g).tolist()
    prompts = [torch.randint(8, cfg_d["vocab_size"], (n,), generator=g).tolist() for n in lens]
    plain = Pipeline(model_dirs["B"], dtype="float32", device=0, page_size=page, max_tokens=2048, max_requests=4)
    plain.runner.use_tapes = False
    plain.runner.use_graphs = False
    want = [plain.apply([p], max_new_tokens=n, do_sample=False, ignore_eos=True)[0] for p, n in zip(prompts, news)]
    assert plain.runner.tape_replays == 0 and plain.runner.graph_replays == 0
    busy = Pipeline(model_dirs["B"], dtype="float32", device=0, page_size=page, max_tokens=20 * page, max_requests=6,
                    max_tokens_per_step=48, chunk=16)
    for rounds in range(2):
        got = []
        for lo in range(0, 24, 8):   # eight at a time, each with its own length to generate
            n = max(news[lo: lo + 8])
            out = busy.apply(prompts[lo: lo + 8], max_new_tokens=n, do_sample=False, ignore_eos=True)
            got += [o[:k] for o, k in zip(out, news[lo: lo + 8])]
        assert got == want
    assert busy.runner.tape_replays > 0 and busy.runner.graph_replays > 0
    assert busy.scheduler.counters["pushed_out"] > 0
    assert busy.runner.cache.groups[0].pool.num_used == 0
