"""Command line in the manner of the reference's main.cpp (flags at main.cpp:7-19, loop at :55-81):

    python -m tiny_llm_b200 --model_path=DIR [--device=0] [--max_new_tokens=256] [--do_sample=true]
        [--temperature=0.7] [--top_k=50] [--top_p=0.95] [--page_mode] [--dtype=bfloat16] [--seed=0]
        [--page_size=16] [--num_pages=N | --max_tokens=N] [--max_requests=4] [--max_tokens_per_step=2048]
        [--chunk=512] [--prompt_per_line]
    python -m tiny_llm_b200 --random_weights --config=CONFIG.json [--seed=0] ...

Flags are gflags-style: --name=value, --name value, --flag / --noflag for booleans.  The tokenizer
is outside the engine, so a prompt is a list of token ids: type ids separated by blanks or commas,
over as many lines as needed; an empty line ends the prompt, end of input exits.  With
--prompt_per_line every line of such a block is a prompt of its own and the block's prompts are
generated together: the scheduler admits them side by side, cuts them into portions of --chunk tokens
under --max_tokens_per_step, and decodes them as one batch.  --random_weights makes a model folder
from a config.json and --seed in a temporary place and runs from it (--seed also seeds the sampler).
--page_mode is accepted for compatibility: the paged cache is the only mode here."""
from __future__ import annotations

import re
import sys
import tempfile

FLAGS = {
    "model_path": (str, "", "Path to the model directory (required)"),
    "device": (int, 0, "CUDA device ID"),
    "max_new_tokens": (int, 256, "Maximum number of tokens to generate"),
    "do_sample": (bool, True, "Whether to use sampling; if false, use greedy decoding"),
    "temperature": (float, 0.7, "Sampling temperature (higher = more creative)"),
    "top_k": (int, 50, "Sample from the top K most likely tokens"),
    "top_p": (float, 0.95, "Sample from the smallest set of tokens whose cumulative probability > p"),
    "page_mode": (bool, True, "Paged attention (always on; accepted for compatibility)"),
    "dtype": (str, "bfloat16", "bfloat16 (serving kernels) or float32 (everything in true 32-bit)"),
    "seed": (int, 0, "Seed of the sampler's random stream"),
    "page_size": (int, 16, "Tokens per cache page"),
    "max_tokens": (int, 0, "Tokens the cache pool holds (0: max_requests x the model's positions)"),
    "num_pages": (int, 0, "Pages of the cache pool (another way to say max_tokens = num_pages x page_size)"),
    "max_requests": (int, 4, "Requests that run side by side (state slots)"),
    "max_tokens_per_step": (int, 2048, "Token budget of one step"),
    "chunk": (int, 0, "Largest portion of a prompt that runs in one step (0: the step's token budget)"),
    "prompt_per_line": (bool, False, "Every line of an input block is a prompt; a block is generated as one batch"),
    "random_weights": (bool, False, "Make the model from --config and --seed instead of reading --model_path"),
    "config": (str, "", "config.json of the model to make with --random_weights"),
}


def _to_bool(s: str) -> bool:
    if s.lower() in ("1", "true", "t", "yes", "y"):
        return True
    if s.lower() in ("0", "false", "f", "no", "n"):
        return False
    raise ValueError(f"not a boolean: {s!r}")


def usage(prog: str) -> str:
    lines = [f"Usage: {prog} --model_path <path> [options]"]
    for name, (typ, default, text) in FLAGS.items():
        lines.append(f"  --{name} ({text}) type: {typ.__name__} default: {default!r}")
    return "\n".join(lines)


def parse_flags(argv):
    values = {k: v[1] for k, v in FLAGS.items()}
    i = 0
    while i < len(argv):
        arg = argv[i]
        if not arg.startswith("-"):
            raise ValueError(f"unexpected argument {arg!r}")
        body = arg.lstrip("-")
        name, eq, val = body.partition("=")
        if name.startswith("no") and name[2:] in FLAGS and FLAGS[name[2:]][0] is bool and not eq:
            values[name[2:]] = False
        elif name not in FLAGS:
            raise ValueError(f"unknown command line flag '{name}'")
        else:
            typ = FLAGS[name][0]
            if typ is bool:
                if eq:
                    values[name] = _to_bool(val)
                elif i + 1 < len(argv) and not argv[i + 1].startswith("-") and argv[i + 1].lower() in (
                        "true", "false", "0", "1", "t", "f", "yes", "no", "y", "n"):
                    i += 1
                    values[name] = _to_bool(argv[i])
                else:
                    values[name] = True
            else:
                if not eq:
                    i += 1
                    if i >= len(argv):
                        raise ValueError(f"flag '--{name}' is missing its argument")
                    val = argv[i]
                values[name] = typ(val)
        i += 1
    return values


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    prog = "python -m tiny_llm_b200"
    if any(a in ("--help", "-h", "-help") for a in argv):
        print(usage(prog))
        return 0
    try:
        f = parse_flags(argv)
    except ValueError as e:
        print(f"ERROR: {e}\n\n{usage(prog)}", file=sys.stderr)
        return 1
    if not f["model_path"] and not f["random_weights"]:
        print("Error: --model_path is mandatory.\n\n" + usage(prog), file=sys.stderr)
        return 1
    if f["random_weights"] and not f["config"]:
        print("Error: --random_weights needs --config.\n\n" + usage(prog), file=sys.stderr)
        return 1
    scratch = None
    try:
        from .engine import Pipeline

        model_path = f["model_path"]
        if f["random_weights"]:
            import torch

            from .config import load_config
            from .weights import write_random_model
            scratch = tempfile.TemporaryDirectory(prefix="tiny_llm_random_")
            model_path = write_random_model(scratch.name, load_config(f["config"]), seed=f["seed"], dtype=torch.float32)
        max_tokens = f["max_tokens"] or f["num_pages"] * f["page_size"] or None
        pipeline = Pipeline(model_path, dtype=f["dtype"], device=f["device"], page_size=f["page_size"],
                            max_tokens=max_tokens, max_requests=f["max_requests"],
                            max_tokens_per_step=f["max_tokens_per_step"], chunk=f["chunk"] or None)
        print("\n>>> [Page Mode] Interactive Mode (Multi-line enabled) <<<")
        print(">>> Enter your prompt as token ids. Enter a blank line to end the current input. "
              "Enter EOF (Ctrl+D) to exit. <<<")
        while True:
            print("\n[Input] >", flush=True)
            buf = []
            eof = False
            while True:
                line = sys.stdin.readline()
                if line == "":
                    eof = True
                    break
                if line.strip() == "":
                    break
                buf.append(line)
            if eof and not buf:
                break
            blocks = buf if f["prompt_per_line"] else [" ".join(buf)]
            prompts = [[int(t) for t in re.split(r"[\s,]+", b.strip()) if t] for b in blocks]
            prompts = [p for p in prompts if p]
            if not prompts:
                print("The prompt is empty. Please re-enter.")
                continue
            outs = pipeline.apply(prompts, max_new_tokens=f["max_new_tokens"], do_sample=f["do_sample"],
                                  temperature=f["temperature"], top_k=f["top_k"], top_p=f["top_p"], seed=f["seed"])
            print("[Output] >\n" + "\n".join(" ".join(str(t) for t in out) for out in outs), flush=True)
            if eof:
                break
    except Exception as e:  # the reference reports and exits 1 (main.cpp:82-85)
        print(f"[Fatal]: {e}", file=sys.stderr)
        return 1
    finally:
        if scratch is not None:
            scratch.cleanup()
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
