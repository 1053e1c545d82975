"""Builds replay traces (whole, tail decoded, portions, mixed) and runs them, through bin/trace_run
as a user would or through a runner in this process, and gathers logits per request and position."""
import json
import os
import random
import subprocess
import sys
import tempfile

import numpy as np
import torch

import plain_llama as pl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_requests(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def plain_logits(model_dir, reqs, dtype):
    """Logits [T, V] of every request from the plain implementation, whole and alone."""
    cfg = pl.load_config(model_dir)
    w = pl.load_weights(model_dir)
    quant = pl.no_quant
    if dtype == "bfloat16":
        w = {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in w.items()}
        quant = pl.bf16_quant
    return {rid: pl.forward(cfg, w, toks, quant=quant) for rid, toks in reqs.items()}


def tolerance(ref, dtype, ref32=None):
    """float32: the engine must match to 2e-5 on these small models (1e-4 is the contract at 1.1B size).
    bfloat16: the yardstick is the error that bfloat16 rounding itself causes in the plain
    implementation for this very request, max |plain(bfloat16 roundings) - plain(32-bit)|: the engine
    rounds at the same places, so it must agree with the rounded plain implementation at least as
    well as that.  Without the 32-bit logits at hand: 2^-6 of the largest logit."""
    if dtype == "float32":
        return 2e-5
    if ref32 is not None:
        return float((ref - ref32).abs().max())
    return 2.0 ** -6 * float(ref.abs().max())


# ----------------------------------------------------------------------------- traces
# A trace is a list of steps {"entries": [{"id", "tokens", "want"}], "end": [...]}; request ids get a
# prefix per scenario so that scenarios can share one replay.


def trace_whole(reqs, prefix="w"):
    return [{"entries": [{"id": prefix + rid, "tokens": t, "want": list(range(len(t)))}], "end": [prefix + rid]}
            for rid, t in reqs.items()]


def trace_tail(reqs, tail=32, prefix="t"):
    steps = []
    for rid, t in reqs.items():
        head = max(1, len(t) - tail)
        steps.append({"entries": [{"id": prefix + rid, "tokens": t[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(t)):
            steps.append({"entries": [{"id": prefix + rid, "tokens": [t[i]], "want": [0]}],
                          "end": [prefix + rid] if i == len(t) - 1 else []})
        if head == len(t):
            steps[-1]["end"] = [prefix + rid]
    return steps


def trace_portions(reqs, seed, prefix="p"):
    """Portions of changing size, down to two tokens and one."""
    rng = random.Random(seed)
    steps = []
    for rid, t in reqs.items():
        pos = 0
        sizes = [2, 1, 3, 2]
        while pos < len(t):
            n = sizes.pop(0) if sizes else rng.choice([2, 2, 3, 5, 7, 11, 16, 17, 31])
            n = min(n, len(t) - pos)
            steps.append({"entries": [{"id": prefix + rid, "tokens": t[pos:pos + n], "want": list(range(n))}],
                          "end": [prefix + rid] if pos + n == len(t) else []})
            pos += n
    return steps


def trace_mixed(reqs, seed, max_live=4, prefix="m"):
    """Up to max_live requests at a time: some bring portions of their prompt, others single tokens,
    some sit a step out; a request that ends makes room for the next, so pages are used again."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, t = waiting.pop(0)
            live[rid] = [t, 0, rng.randint(len(t) // 3, max(len(t) // 3, len(t) - 1))]  # tokens, pos, where decoding starts
        entries, end = [], []
        for rid in list(live):
            t, pos, decode_from = live[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step
            n = 1 if pos >= decode_from else min(rng.choice([2, 3, 5, 8, 13, 24]), decode_from - pos)
            n = min(n, len(t) - pos)
            entries.append({"id": prefix + rid, "tokens": t[pos:pos + n], "want": list(range(n))})
            live[rid][1] = pos + n
            if pos + n == len(t):
                end.append(prefix + rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def tokens_needed(steps, round_to=64):
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up to a multiple of 64."""
    held, most = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def gather(steps, outputs, vocab):
    """outputs[i]: array [wanted, V] of step i (or None) -> {request id: tensor [T, V]} (wanted rows in order)."""
    rows = {}
    for s, out in zip(steps, outputs):
        k = 0
        for e in s["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(torch.from_numpy(np.array(out[k], dtype=np.float32)))
                k += 1
        assert out is None and k == 0 or k == out.shape[0]
    return {rid: torch.stack(r) for rid, r in rows.items()}


# ----------------------------------------------------------------------------- running


def run_trace_cli(model_dir, dtype, steps, vocab, max_tokens=None, page_size=None, env=None):
    """Feeds the steps to bin/trace_run one by one, waiting for `done <step>` after each."""
    max_tokens = tokens_needed(steps) if max_tokens is None else max_tokens
    with tempfile.TemporaryDirectory() as out:
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
               "--out", out, "--max-tokens", str(max_tokens)]
        if page_size:
            cmd += ["--page-size", str(page_size)]
        proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        try:
            for i, s in enumerate(steps):
                proc.stdin.write(json.dumps({"step": i, "entries": s["entries"], "end": s["end"]}) + "\n")
                proc.stdin.flush()
                line = proc.stdout.readline().strip()
                assert line == f"done {i}", f"trace_run answered {line!r} at step {i}"
            proc.stdin.close()
            assert proc.wait(timeout=120) == 0
        finally:
            if proc.poll() is None:
                proc.kill()
        outputs = []
        for i, s in enumerate(steps):
            path = os.path.join(out, f"{i}.f32")
            wanted = sum(len(e["want"]) for e in s["entries"])
            if wanted:
                arr = np.fromfile(path, dtype="<f4")
                assert arr.size == wanted * vocab, (i, arr.size, wanted, vocab)
                outputs.append(arr.reshape(wanted, vocab))
            else:
                assert not os.path.exists(path)
                outputs.append(None)
    return gather(steps, outputs, vocab)


def run_trace_runner(runner, steps, vocab):
    """The same replay through a ModelRunner in this process."""
    from tiny_llm_b200.engine import StepEntry

    outputs = []
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not runner.cache.has_request(e["id"]):
                assert runner.cache.add_request(e["id"]) is not None
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = runner.step(entries)
        outputs.append(None if logits is None else logits.detach().cpu().numpy().copy())
        for rid in s["end"]:
            runner.cache.free_request(rid)
        runner.cache.check()
    return gather(steps, outputs, vocab)


def compare(got, ref, prefix, dtype, what, ref32=None):
    """`ref`: the plain implementation's logits in the path's precision; `ref32`: its 32-bit logits
    (the bfloat16 yardstick, see tolerance())."""
    worst = 0.0
    for rid, r in ref.items():
        g = got[prefix + rid]
        assert g.shape == r.shape, (what, rid, g.shape, r.shape)
        diff = (g - r).abs()
        tol = tolerance(r, dtype, None if ref32 is None else ref32[rid])
        if float(diff.max()) > tol:
            bad = (diff.max(dim=1).values > tol).nonzero().flatten()
            raise AssertionError(f"{what}: request {rid} differs from the plain implementation first at position "
                                 f"{int(bad[0])} of {r.shape[0]} (max |diff| {float(diff.max()):.3e}, tolerance {tol:.3e}; "
                                 f"wrong positions: {bad.tolist()[:20]})")
        worst = max(worst, float(diff.max()) / tol)
    record_margin(what, dtype, worst)
    return worst


def record_margin(what, dtype, worst, tolerance_kind="|diff| / tolerance"):
    """Prints how much of its tolerance a comparison used and, when TLLM_MARGIN_FILE names a file,
    appends the figure there as a JSON line, so that a run leaves a record of its margins."""
    print(f"[margin] {what} {dtype}: worst {tolerance_kind} = {worst:.3g}")
    path = os.environ.get("TLLM_MARGIN_FILE")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"what": what, "dtype": dtype, "kind": tolerance_kind, "worst": float(f"{worst:.4g}")}) + "\n")
