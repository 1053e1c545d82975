#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, TinyLlama-1.1B layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A step is one decode step of a batch of 8 requests at a context of 2,048 tokens (the last timed step
writes position 2047).  `value` is decoded tokens per second with the device clock around K steps
that are enqueued back to back; `e2e` is the same through the Python entry point with host tokens in
and out every step.  The line also carries a 2,048-token prefill, decoding at batch 1 and 64, the
HBM roofline of the decode step, and the clocks seen while timing."""
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
CONTEXT = 2048
BATCH = 8
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
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


def build_model(layers, dtype, device):
    import torch
    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state, random_state
    cfg = LlamaConfig.from_dict(dict(TINYLLAMA, num_hidden_layers=layers))
    model = DecoderModel(cfg.model_spec())
    specs = model.weight_specs()
    state = random_state(specs, 2, cfg.initializer_range, dtype, device=device)   # seed 2, N(0, 0.02)
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


def timed_decode(runner, batch, start_len, steps, warmup, sampler_out):
    """Prefills `batch` requests to start_len tokens, then runs warmup + steps decode steps enqueued
    back to back; returns (ms per step over the timed steps, kernels launched in them)."""
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
    feed = torch.randint(0, vocab, (warmup + steps, batch), generator=g).tolist()

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(rids)])
        ops.argmax(logits, sampler_out[:batch])

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    before = ops.launches
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(warmup, warmup + steps):
        if TRACE and i == warmup + steps - 1:   # the last step alone, between two reads of the timeline notes
            torch.cuda.synchronize()
            ops.trace_dump()
        one(i)
    t1.record()
    torch.cuda.synchronize()
    if TRACE:
        timed_decode.timeline = ops.trace_dump()
    ms = t0.elapsed_time(t1) / steps
    launched = ops.launches - before
    for rid in rids:
        runner.cache.free_request(rid)
    return ms, launched


def timed_prefill(runner, tokens, repeats=5):
    import torch
    from tiny_llm_b200.engine import StepEntry
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, runner.model.spec.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(repeats + 2):
        runner.cache.add_request("p")
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry("p", toks, [tokens - 1])])
        t1.record()
        torch.cuda.synchronize()
        runner.cache.free_request("p")
        if i >= 2:
            times.append(t0.elapsed_time(t1))
    return statistics.median(times)


def timed_e2e(pipe, batch, context, steps, warmup):
    """The same decode through the Python entry point: host tokens in and out every step.  The
    requests are admitted over several steps (the prompt budget), so they get a margin of tokens
    that keeps all of them decoding side by side through warm-up and the timed steps; the last timed
    step still runs within `margin` tokens of `context`."""
    import torch
    from tiny_llm_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(3)
    vocab = pipe.model.spec.vocab_size
    margin = 2 * batch + 4
    new_tokens = steps + warmup + margin
    params = SamplingParams(max_new_tokens=new_tokens, do_sample=False, ignore_eos=True)
    for _ in range(batch):
        pipe.add_request(torch.randint(0, vocab, (context - new_tokens,), generator=g).tolist(), params)
    while any(r.remaining > 1 for r in pipe.scheduler.running) or pipe.scheduler.waiting:
        pipe.step()                                  # prompts in (untimed)
    for _ in range(warmup):
        pipe.step()
    torch.cuda.synchronize()
    assert len(pipe.scheduler.running) == batch
    t0 = time.perf_counter()
    for _ in range(steps):
        pipe.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert len(pipe.scheduler.running) == batch      # nobody ended inside the timed steps
    while pipe.has_work():
        pipe.step()
    return dt * 1e3 / steps


def reference_arm():
    """The reference is a Bazel + Rust + CUDA >= 13 C++ project without a Python package: the one
    allowed offline install (pip install --no-index ... of the reference checkout) has nothing to build."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "zscey/tiny-llm is a Bazel/Rust/CUDA-13 C++ project with no setup.py or pyproject.toml; "
                      "pip cannot install it offline and no Bazel or Rust toolchain exists here"}))
    return 0


def main():
    global PAGE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=TINYLLAMA["num_hidden_layers"],
                    help="fewer layers than the model has (layer sizes stay); both numbers are reported")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only (for profiler captures of a small case)")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests of the decode step (default 8)")
    ap.add_argument("--page-size", type=int, default=PAGE, help="tokens per page of the cache")
    args = ap.parse_args()
    PAGE = args.page_size
    if args.impl == "reference":
        return reference_arm()
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
    cfg, model = build_model(args.layers, dtype, device)
    itemsize = 2 if dtype == torch.bfloat16 else 4
    start_len = CONTEXT - (steps + warmup)            # the last timed step writes position CONTEXT - 1
    runner = make_runner(model, dtype, device, max_tokens=64 * CONTEXT, page_size=PAGE, max_requests=64,
                         max_tokens_per_step=2048)
    out = torch.zeros(64, dtype=torch.int32, device=device)

    if args.only != "all":
        # a small, single-purpose run for a profiler capture: one plain line, no record
        if args.only == "decode":
            ms, launched = timed_decode(runner, args.batch, start_len, steps, warmup, out)
            rec = {"only": "decode", "batch": args.batch, "layers": args.layers, "ms_per_step": round(ms, 4),
                   "gpu_launches": launched}
            if TRACE:
                rec["timeline"] = timeline_summary(timed_decode.timeline)
            print(json.dumps(rec))
        else:
            ops.attention_tc_timing()   # (a build with cycle counters: start from zero)
            rec = {"only": "prefill", "layers": args.layers, "tokens": 2048,
                   "ms": round(timed_prefill(runner, 2048, repeats=2), 3)}
            cycles = ops.attention_tc_timing()
            if cycles is not None:
                # cycles per key tile in the roles of the attention kernel's first CTA, which walks 2048 / 64 tiles
                tiles = (2048 // 64) * args.layers * 4
                rec["attention_cycles_per_tile"] = {n: round(v / tiles, 1) for n, v in cycles.items()}
            print(json.dumps(rec))
        return 0

    sampler = ClockSampler().start()
    ms, launched = timed_decode(runner, BATCH, start_len, steps, warmup, out)
    clocks = sampler.stop()

    points = {}
    for b, key in ((1, "decode_b1"), (64, "decode_b64")):
        s = min(steps, 32)
        pms, _ = timed_decode(runner, b, CONTEXT - (s + 3), s, 3, out)
        points[key] = round(b * 1e3 / pms, 1)
    prefill_ms = timed_prefill(runner, 2048)

    pipe = Pipeline.from_model(cfg, model, dtype=dtype, device=0, page_size=PAGE, max_tokens=BATCH * CONTEXT,
                               max_requests=BATCH, max_tokens_per_step=2048, chunk=1024)
    e2e_ms = timed_e2e(pipe, BATCH, CONTEXT, steps, warmup)
    h2d = 4 * (3 * BATCH + (BATCH + 1) + 3 * BATCH + BATCH + BATCH + BATCH * pipe.runner.max_blocks)

    # roofline of the decode step: every weight once + the cache of the live requests
    kv_per_token = sum(g.bytes_per_token(itemsize) for g in runner.cache.groups)
    mean_ctx = start_len + warmup + (steps + 1) / 2.0
    step_bytes = weight_bytes(model) + BATCH * mean_ctx * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9
    # flops of the prefill step: 2 * T * matrix parameters + causal attention + LM head on one row
    s = model.spec
    c = cfg
    per_layer = (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim +
                 c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    t = 2048
    flops = 2.0 * t * per_layer * args.layers + 2.0 * t * t * c.num_attention_heads * c.head_dim * args.layers + \
        2.0 * c.hidden_size * c.vocab_size
    peak_flops = pk["bf16_tflops"] * 1e12 if dtype == torch.bfloat16 else None
    value = BATCH * 1e3 / ms
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
                   "peaks": pk["source"]},
        "e2e": {"value": round(BATCH * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * BATCH},
        "gpu_launches": launched,
        "prefill": {"value": round(t * 1e3 / prefill_ms, 1), "tokens": t, "ms": round(prefill_ms, 3),
                    "frac": None if peak_flops is None else round(flops / (prefill_ms * 1e-3) / peak_flops, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "clocks": clocks,
        "libraries": sorted(os.path.basename(p) for p in ops.build.loaded_libraries().values()),
    }
    ops.check_status()   # no kernel of the timed runs gave up a bounded wait
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
