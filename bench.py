#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, TinyLlama-1.1B layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A step is one decode step of a batch of 8 requests at a context of 2,048 tokens (the last timed step
writes position 2047).  `value` is decoded tokens per second with the device clock around K steps
that are enqueued back to back; `e2e` is the same through the Python entry point with host tokens in
and out every step.  Every figure is the median of REPEATS timed regions of K steps each inside the
one run.  The line also carries a 2,048-token prefill, decoding at batch 1 and 64, the stated workload
of the model's benchmark (512-token prompts + 256 generated tokens through the entry point, admission and
prompts included), the same points at the Llama-2-7B and Llama-3-8B layer sizes (all 32 layers), the HBM
roofline of every decode point, and the clocks seen while timing."""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TINYLLAMA = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=22, hidden_size=2048,
                 num_attention_heads=32, num_key_value_heads=4, intermediate_size=5632, vocab_size=32000,
                 rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=2048, tie_word_embeddings=False,
                 hidden_act="silu", initializer_range=0.02, torch_dtype="bfloat16")
LLAMA2_7B = dict(TINYLLAMA, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=32,
                 intermediate_size=11008, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096)
LLAMA3_8B = dict(TINYLLAMA, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                 intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192)
OTHER_SHAPES = {"llama2_7b": (LLAMA2_7B, 3), "llama3_8b": (LLAMA3_8B, 4)}   # configuration, seed of its weights
CONTEXT = 2048
BATCH = 8
PAGE = 16
REPEATS = 5
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.rows = []
        self.proc = None
        self.device = device

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)

    def stop(self):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(int(r[0]) for r in self.rows)), "sm_max_mhz": int(self.rows[0][1]),
                "reasons": reasons, "samples": len(self.rows)}


def build_model(layers, dtype, device, shape=TINYLLAMA, seed=2):
    import torch
    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state, random_state
    cfg = LlamaConfig.from_dict(dict(shape, num_hidden_layers=layers))
    model = DecoderModel(cfg.model_spec())
    specs = model.weight_specs()
    state = random_state(specs, seed, cfg.initializer_range, dtype, device=device)   # N(0, 0.02)
    model.load(load_state(specs, state, dtype, device))
    return cfg, model


def weight_bytes(model):
    """Bytes of every weight a decode step reads once: all matrices and norm vectors, not the
    embedding table (its rows are gathered)."""
    seen, total = set(), 0
    tensors = [model.lm_head, model.final_norm.weight]
    for b in model.blocks:
        tensors += [b.norm1.weight, b.norm2.weight, b.mixer.w_qkv, b.mixer.w_o, b.ffn.w_gate_up, b.ffn.w_down]
    for t in tensors:
        if t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    return total


TRACE = os.environ.get("TLLM_TRACE") == "1"   # kernels built with timeline notes (a build for measurements)


def timeline_summary(records):
    """Per kind of launch (library, grid, block): how many, and the mean time in us from the moment the
    kernel before it had finished to the moment it had finished itself, inside the replayed graph."""
    kinds = {}
    for i, r in enumerate(records[:-1]):
        name = f"{r[6]} grid {r[2]}x{r[3]}x{r[4]} block {r[5]}"
        k = kinds.setdefault(name, [0, 0.0])
        k[0] += 1
        k[1] += (records[i + 1][1] - r[1]) / 1e3
    out = {n: {"launches": c, "mean_us": round(t / c, 2), "total_us": round(t, 1)} for n, (c, t) in kinds.items()}
    return dict(sorted(out.items(), key=lambda kv: -kv[1]["total_us"]))


def timed_decode(runner, batch, start_len, steps, warmup, sampler_out, repeats=1):
    """Prefills `batch` requests to start_len tokens, then runs warmup + repeats x steps decode steps enqueued
    back to back, each run of `steps` between two events; returns (median ms per step over the runs,
    kernels launched in one run, mean context of the timed steps)."""
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import StepEntry
    g = torch.Generator().manual_seed(0)
    vocab = runner.model.spec.vocab_size
    rids = [f"d{batch}_{i}" for i in range(batch)]
    for rid in rids:
        assert runner.cache.add_request(rid) is not None
        toks = torch.randint(0, vocab, (start_len,), generator=g).tolist()
        for lo in range(0, start_len, 1024):
            runner.step([StepEntry(rid, toks[lo: lo + 1024], [])])
    feed = torch.randint(0, vocab, (warmup + repeats * steps, batch), generator=g).tolist()

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(rids)])
        ops.argmax(logits, sampler_out[:batch])

    for i in range(warmup):
        one(i)
    times, launched = [], 0
    for rep in range(repeats):
        torch.cuda.synchronize()
        before = ops.launches
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(warmup + rep * steps, warmup + (rep + 1) * steps):
            if TRACE and rep == repeats - 1 and i == warmup + repeats * steps - 1:   # the last step alone, between two reads of the timeline notes
                torch.cuda.synchronize()
                ops.trace_dump()
            one(i)
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) / steps)
        launched = ops.launches - before
    if TRACE:
        timed_decode.timeline = ops.trace_dump()
    for rid in rids:
        runner.cache.free_request(rid)
    mean_ctx = start_len + warmup + (repeats * steps + 1) / 2.0
    return statistics.median(times), launched, mean_ctx


def timed_prefill(runner, tokens, repeats=5):
    import torch
    from tiny_llm_b200.engine import StepEntry
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, runner.model.spec.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(repeats + 2):
        runner.cache.add_request("p")
        torch.cuda.synchronize()
        if TRACE and i == repeats + 1:   # the last step alone, between two reads of the timeline notes
            from tiny_llm_b200 import ops
            ops.trace_dump()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry("p", toks, [tokens - 1])])
        t1.record()
        torch.cuda.synchronize()
        if TRACE and i == repeats + 1:
            timed_prefill.timeline = ops.trace_dump()
        runner.cache.free_request("p")
        if i >= 2:
            times.append(t0.elapsed_time(t1))
    return statistics.median(times)


def timed_e2e(pipe, batch, context, steps, warmup, repeats=1):
    """The same decode through the Python entry point: host tokens in and out every step.  The
    requests are admitted over several steps (the prompt budget), so they get a margin of tokens
    that keeps all of them decoding side by side through warm-up and the timed steps; the last timed
    step still runs within `margin` tokens of `context`.  Returns the median over `repeats` runs of
    `steps` steps each of the wall time per step."""
    import torch
    from tiny_llm_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(3)
    vocab = pipe.model.spec.vocab_size
    margin = 2 * batch + 4
    new_tokens = repeats * steps + warmup + margin
    params = SamplingParams(max_new_tokens=new_tokens, do_sample=False, ignore_eos=True)
    for _ in range(batch):
        pipe.add_request(torch.randint(0, vocab, (context - new_tokens,), generator=g).tolist(), params)
    while any(r.remaining > 1 for r in pipe.scheduler.running) or pipe.scheduler.waiting:
        pipe.step()                                  # prompts in (untimed)
    for _ in range(warmup):
        pipe.step()
    times = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        assert len(pipe.scheduler.running) == batch
        t0 = time.perf_counter()
        for _ in range(steps):
            pipe.step()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3 / steps)
        assert len(pipe.scheduler.running) == batch      # nobody ended inside the timed steps
    timed_e2e.h2d_bytes = pipe.runner.last_h2d_bytes     # of a timed step: tokens, positions, request and block tables
    while pipe.has_work():
        pipe.step()
    return statistics.median(times)


def timed_workload(pipe, batch, prompt_len=512, new_tokens=256, repeats=3):
    """The benchmark's stated workload through the entry point: `batch` requests of a 512-token random
    prompt each, 256 tokens generated greedily, from the first add_request to the last token on the
    host (admission, prompts in portions, decoding).  Returns generated tokens per second of wall time,
    median of `repeats` runs (after one untimed run)."""
    import torch
    g = torch.Generator().manual_seed(4)
    vocab = pipe.model.spec.vocab_size
    rates = []
    for rep in range(repeats + 1):
        prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in range(batch)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = pipe.apply(prompts, max_new_tokens=new_tokens, do_sample=False, ignore_eos=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert all(len(o) == new_tokens for o in out)
        if rep:
            rates.append(batch * new_tokens / dt)
    return statistics.median(rates)


def decode_bytes(model, runner, batch, mean_ctx, itemsize):
    """Bytes a decode step has to read: every weight once and the cache of the live requests."""
    kv_per_token = sum(g.bytes_per_token(itemsize) for g in runner.cache.groups)
    return weight_bytes(model) + batch * mean_ctx * kv_per_token


def prefill_flops(c, layers, t):
    """2 * T * matrix parameters + causal attention + LM head on one row."""
    per_layer = (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim +
                 c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    return 2.0 * t * per_layer * layers + 2.0 * t * t * c.num_attention_heads * c.head_dim * layers + \
        2.0 * c.hidden_size * c.vocab_size


def other_shape_points(name, shape, seed, dtype, device, pk, steps, out, points, fracs):
    """Decode at batch 16 and 64 and a 2,048-token prefill at another model's layer sizes, all of its layers."""
    import gc

    import torch
    from tiny_llm_b200.engine import make_runner
    cfg, model = build_model(shape["num_hidden_layers"], dtype, device, shape=shape, seed=seed)
    itemsize = 2 if dtype == torch.bfloat16 else 4
    runner = make_runner(model, dtype, device, max_tokens=64 * CONTEXT, page_size=PAGE, max_requests=64,
                         max_tokens_per_step=2048)
    s = min(steps, 16)
    for b in (16, 64):
        ms, _, ctx = timed_decode(runner, b, CONTEXT - (3 * s + 3), s, 3, out, repeats=3)
        points[f"{name}_decode_b{b}"] = round(b * 1e3 / ms, 1)
        fracs[f"{name}_decode_b{b}"] = round(decode_bytes(model, runner, b, ctx, itemsize) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    long_ctx = min(cfg.max_position_embeddings, 8192)
    if long_ctx > CONTEXT:   # a longer context where the model has the positions: 16 requests at 8,192 tokens
        ms, _, ctx = timed_decode(runner, 16, long_ctx - (3 * s + 3), s, 3, out, repeats=3)
        points[f"{name}_decode_b16_ctx{long_ctx}"] = round(16 * 1e3 / ms, 1)
        fracs[f"{name}_decode_b16_ctx{long_ctx}"] = round(decode_bytes(model, runner, 16, ctx, itemsize) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    ms = timed_prefill(runner, 2048, repeats=3)
    points[f"{name}_prefill_2048"] = round(2048 * 1e3 / ms, 1)
    if dtype == torch.bfloat16:
        fracs[f"{name}_prefill_2048"] = round(prefill_flops(cfg, cfg.num_hidden_layers, 2048) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
    del runner, model
    gc.collect()
    torch.cuda.empty_cache()


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_arm(steps, warmup):
    """The reference arm: zscey/tiny-llm's own engine, unmodified (its parser, plan, runtime and CUDA kernels,
    compiled by baseline/build_reference.py and driven below the tokenizer by baseline/ref_driver.cpp as its
    Pipeline::apply drives it), at the same configuration: TinyLlama-1.1B layer sizes, 22 layers, batch 8,
    context 2,048, paged mode, greedy sampling on the host.  Its only dtype is float32.  pip cannot install
    the reference (no setup.py or pyproject.toml: a Bazel + Rust project), so the arm is built from its sources."""
    import tempfile
    exe = os.path.join(REF_DIR, "ref_driver")
    if not os.path.isfile(exe):
        try:
            res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py")],
                                 capture_output=True, text=True, timeout=1500)
            why = (res.stderr.strip().splitlines() or res.stdout.strip().splitlines() or ["?"])[-1]
        except (OSError, subprocess.TimeoutExpired) as e:
            why = str(e)
        if not os.path.isfile(exe):
            print(json.dumps({"impl": "reference", "unavailable": f"the reference could not be built here: {why}"[:300]}))
            return 0
    cfg = dict(TINYLLAMA, torch_dtype="float32", eos_token_id=None, attention_bias=False, rope_scaling=None)
    pk = peaks()

    def run(mode, *extra):
        with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
            json.dump(cfg, f)
        try:
            res = subprocess.run([exe, mode, "--config", f.name] + [str(x) for x in extra], capture_output=True, text=True, timeout=900)
        finally:
            os.unlink(f.name)
        if res.returncode != 0:
            raise RuntimeError((res.stderr.strip().splitlines() or ["ref_driver failed"])[-1])
        return json.loads(res.stdout.strip().splitlines()[-1])

    try:
        sampler = ClockSampler().start()
        main_run = run("bench", "--batch", BATCH, "--context", CONTEXT, "--steps", steps, "--warmup", warmup, "--repeats", REPEATS)
        clocks = sampler.stop()
        s = min(steps, 8)
        points, notes = {}, {}
        for b in (1, 16, 64):
            try:
                r = run("bench", "--batch", b, "--context", CONTEXT, "--steps", s, "--warmup", 3, "--repeats", 3)
                points[f"decode_b{b}"] = round(b * 1e3 / r["ms_per_step_device"], 1)
            except RuntimeError as e:   # (at batch 64 the reference's own memory planner gives up: "Bad virtual block.")
                points[f"decode_b{b}"] = None
                notes[f"decode_b{b}"] = f"the reference does not run this batch: {e}"[:200]
        pre = run("prefill", "--tokens", 2048, "--repeats", 3)
    except (RuntimeError, OSError, subprocess.TimeoutExpired, ValueError) as e:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's engine did not run: {e}"[:300]}))
        return 0
    ms = main_run["ms_per_step_device"]
    weights = 4 * sum((TINYLLAMA["hidden_size"] * (TINYLLAMA["num_attention_heads"] + 2 * TINYLLAMA["num_key_value_heads"]) * 64 +
                       TINYLLAMA["hidden_size"] ** 2 + 3 * TINYLLAMA["hidden_size"] * TINYLLAMA["intermediate_size"]
                       for _ in range(TINYLLAMA["num_hidden_layers"]))) + 4 * TINYLLAMA["hidden_size"] * TINYLLAMA["vocab_size"]
    kv_per_token = 2 * TINYLLAMA["num_hidden_layers"] * TINYLLAMA["num_key_value_heads"] * 64 * 4
    mean_ctx = CONTEXT - (REPEATS * steps) / 2.0
    achieved = (weights + BATCH * mean_ctx * kv_per_token) / (ms * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8, context 2048 (TinyLlama-1.1B layer sizes)",
        "value": round(BATCH * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic", "impl": "reference",
        "config": {"model": "TinyLlama-1.1B shape, random weights", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": 22, "layers_of_model": 22, "hidden_size": 2048, "heads": 32,
                   "kv_heads": 4, "head_dim": 64, "intermediate_size": 5632, "vocab_size": 32000, "page_size": 32,
                   "same_config": "sizes, batch and context as the other arm; float32 is the reference's only dtype, "
                                  "32 tokens its only page size", "peaks": pk["source"], "repeats": REPEATS,
                   "built_from": "unmodified tiny_llm/ sources, nvcc -arch=sm_100, driven by baseline/ref_driver.cpp"},
        "e2e": {"value": round(BATCH * 1e3 / main_run["ms_per_step_wall"], 1), "unit": "tokens/s",
                "ms_per_step": round(main_run["ms_per_step_wall"], 4), "h2d_bytes_per_step": main_run["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main_run["d2h_bytes_per_step"]},
        "gpu_launches": None,
        "prefill": {"value": round(2048 * 1e3 / pre["ms"], 1), "tokens": 2048, "ms": round(pre["ms"], 3), "frac": None},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_note": notes, "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


def main():
    global PAGE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=TINYLLAMA["num_hidden_layers"],
                    help="fewer layers than the model has (layer sizes stay); both numbers are reported")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only (for profiler captures of a small case)")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests of the decode step (default 8)")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of the prompt step of --only prefill (default 2,048)")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="context the last timed step of --only decode reaches (default 2,048; at most the model's positions)")
    ap.add_argument("--page-size", type=int, default=PAGE, help="tokens per page of the cache")
    ap.add_argument("--shape", default="tinyllama", choices=["tinyllama"] + list(OTHER_SHAPES),
                    help="layer sizes for --only runs (profiler captures of the other models' kernels)")
    ap.add_argument("--quick", action="store_true",
                    help="leave out the workload points and the Llama-2-7B / Llama-3-8B layer sizes")
    args = ap.parse_args()
    PAGE = args.page_size
    if args.impl == "reference":
        return reference_arm(max(1, args.steps), max(3, args.warmup))
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    from tiny_llm_b200 import Pipeline, ops
    from tiny_llm_b200.engine import make_runner, parse_dtype
    dtype = parse_dtype(args.dtype)
    device = "cuda:0"
    torch.cuda.set_device(0)
    pk = peaks()
    if args.shape != "tinyllama" and args.only == "all":
        print("--shape goes with --only decode|prefill (the full run measures every shape)")
        return 2
    shape, seed = (TINYLLAMA, 2) if args.shape == "tinyllama" else OTHER_SHAPES[args.shape]
    cfg, model = build_model(min(args.layers, shape["num_hidden_layers"]), dtype, device, shape=shape, seed=seed)
    itemsize = 2 if dtype == torch.bfloat16 else 4
    start_len = CONTEXT - (REPEATS * steps + warmup)   # the last timed step writes position CONTEXT - 1
    if start_len < 64:
        print(f"--steps {steps} x {REPEATS} repeats + --warmup {warmup} do not fit a context of {CONTEXT}")
        return 2
    if args.only == "decode" and not 64 + steps + warmup <= args.context <= cfg.max_position_embeddings:
        print(f"--context {args.context}: the model has {cfg.max_position_embeddings} positions, and {steps} + {warmup} steps must fit")
        return 2
    pool_tokens = 64 * CONTEXT if args.only != "decode" else max(args.batch, 1) * (args.context + PAGE)
    runner = make_runner(model, dtype, device, max_tokens=pool_tokens, page_size=PAGE, max_requests=64,
                         max_tokens_per_step=2048)
    out = torch.zeros(64, dtype=torch.int32, device=device)

    if args.only != "all":
        # a small, single-purpose run for a profiler capture or a sweep: one plain line, no record
        if args.only == "decode":
            ms, launched, ctx = timed_decode(runner, args.batch, args.context - (steps + warmup), steps, warmup, out)
            moved = decode_bytes(model, runner, args.batch, ctx, itemsize)
            rec = {"only": "decode", "shape": args.shape, "batch": args.batch, "context": args.context,
                   "layers": cfg.num_hidden_layers, "ms_per_step": round(ms, 4),
                   "tokens_per_s": round(args.batch * 1e3 / ms, 1),
                   "hbm_frac": round(moved / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4), "gpu_launches": launched}
            if TRACE:
                rec["timeline"] = timeline_summary(timed_decode.timeline)
            print(json.dumps(rec))
        else:
            ops.attention_tc_timing(cfg.head_dim)   # (a build with cycle counters: start from zero)
            rec = {"only": "prefill", "shape": args.shape, "layers": cfg.num_hidden_layers, "tokens": args.tokens,
                   "ms": round(timed_prefill(runner, args.tokens, repeats=2), 3)}
            if TRACE:
                rec["timeline"] = timeline_summary(timed_prefill.timeline)
            cycles = ops.attention_tc_timing(cfg.head_dim)
            if cycles is not None:
                # cycles per key tile in the roles of the attention kernel's first CTA, which walks 2048 / 64 tiles
                tiles = (args.tokens // 64) * args.layers * 4
                rec["attention_cycles_per_tile"] = {n: round(v / tiles, 1) for n, v in cycles.items()}
            print(json.dumps(rec))
        return 0

    sampler = ClockSampler().start()
    ms, launched, mean_ctx = timed_decode(runner, BATCH, start_len, steps, warmup, out, repeats=REPEATS)
    clocks = sampler.stop()
    achieved = decode_bytes(model, runner, BATCH, mean_ctx, itemsize) / (ms * 1e-3) / 1e9

    points, fracs = {}, {}
    for b, key in ((1, "decode_b1"), (64, "decode_b64")):
        s = min(steps, 32)
        pms, _, ctx = timed_decode(runner, b, CONTEXT - (REPEATS * s + 3), s, 3, out, repeats=REPEATS)
        points[key] = round(b * 1e3 / pms, 1)
        fracs[key] = round(decode_bytes(model, runner, b, ctx, itemsize) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    prefill_ms = timed_prefill(runner, 2048)
    if not args.quick and dtype == torch.bfloat16:
        # shorter prompt steps: fewer tiles than SMs in every product
        for tt in (512, 1024):
            pms = timed_prefill(runner, tt, repeats=3)
            points[f"prefill_{tt}"] = round(tt * 1e3 / pms, 1)
            fracs[f"prefill_{tt}"] = round(prefill_flops(cfg, args.layers, tt) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)

    pipe = Pipeline.from_model(cfg, model, dtype=dtype, device=0, page_size=PAGE, max_tokens=BATCH * CONTEXT,
                               max_requests=BATCH, max_tokens_per_step=2048, chunk=1024)
    e2e_ms = timed_e2e(pipe, BATCH, CONTEXT, steps, warmup, repeats=REPEATS)
    h2d = timed_e2e.h2d_bytes
    del pipe

    # the stated workload of the model's benchmark: 512-token prompts + 256 generated tokens through the entry
    # point (generated tokens per second of wall time for the whole call, prompts and admission included)
    if not args.quick:
        for b in (1, 8, 64):
            wl = Pipeline.from_model(cfg, model, dtype=dtype, device=0, page_size=PAGE, max_tokens=b * 768 + 64,
                                     max_requests=b, max_tokens_per_step=2048, chunk=512)
            points[f"workload_512p_256g_b{b}"] = round(timed_workload(wl, b), 1)
            del wl

    c = cfg
    t = 2048
    flops = prefill_flops(c, args.layers, t)
    peak_flops = pk["bf16_tflops"] * 1e12 if dtype == torch.bfloat16 else None
    value = BATCH * 1e3 / ms
    if not args.quick:
        # the other shapes the benchmark names, all of their layers; this model's tensors go first
        del runner, model
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for name, (shape, seed) in OTHER_SHAPES.items():
            other_shape_points(name, shape, seed, dtype, device, pk, steps, out, points, fracs)
    line = {
        "metric": "decode tok/s at batch 8, context 2048 (TinyLlama-1.1B layer sizes)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": "TinyLlama-1.1B shape, random weights seed 2", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_of_model": TINYLLAMA["num_hidden_layers"],
                   "hidden_size": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate_size": c.intermediate_size, "vocab_size": c.vocab_size,
                   "page_size": PAGE, "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": pk["source"], "repeats": REPEATS, "other_shapes": "llama2_7b and llama3_8b: 32 of 32 layers"},
        "e2e": {"value": round(BATCH * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * (BATCH + 1)},
        "gpu_launches": launched,
        # frac: of the burst peak of a library product timed alone; frac_of_sustained: of what the same product holds
        # back to back under the power cap, which is the state of the GPU inside a step of thousands of tokens
        "prefill": {"value": round(t * 1e3 / prefill_ms, 1), "tokens": t, "ms": round(prefill_ms, 3),
                    "frac": None if peak_flops is None else round(flops / (prefill_ms * 1e-3) / peak_flops, 4),
                    "frac_of_sustained": None if peak_flops is None else
                    round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_frac": fracs, "clocks": clocks,
        "libraries": sorted(os.path.basename(p) for p in ops.build.loaded_libraries().values()),
    }
    ops.check_status()   # no kernel of the timed runs gave up a bounded wait
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
