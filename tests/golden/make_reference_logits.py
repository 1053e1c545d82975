"""Whole-model golden logits from zscey/tiny-llm itself.

Runs the reference's own engine (its parser, plan, runtime and CUDA kernels, unmodified, driven below
the tokenizer by baseline/ref_driver.cpp; built by baseline/build_reference.py) on the two tiny test
configurations with the weights that `write_random_model` makes for them, and stores what it computes:
for a short prompt run whole and a few tokens decoded greedily one by one, the float32 logits of the
prompt's last position and of every decoded position, and the ids it chose.  The reference always wants
an output matrix (tiny_llm/parser/llama_parser.cpp:264-271), so the tied configuration B gets a copy of
its embedding table under lm_head.weight.  Needs a CUDA device.

Usage:  python tests/golden/make_reference_logits.py        (writes tests/golden/reference_logits.safetensors)
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from conftest import TINY  # noqa: E402
from tiny_llm_b200.config import LlamaConfig  # noqa: E402
from tiny_llm_b200.weights import SafetensorsFile, save_safetensors, write_random_model  # noqa: E402

PROMPTS = {"A": [9, 8, 7, 200, 31, 77, 5, 140, 6, 23, 101], "B": [300, 4, 17, 250, 9, 33, 371, 2, 64, 8, 199, 54, 120]}
DECODE = 6


def main():
    driver = os.path.join(ROOT, "baseline", "_ref", "ref_driver")
    if not os.path.isfile(driver):
        raise SystemExit("build the reference first: python baseline/build_reference.py")
    out = {}
    meta = {}
    for name in ("A", "B"):
        cfg_d, _page, seed = TINY[name]
        cfg = LlamaConfig.from_dict(cfg_d)
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, cfg, seed=seed, dtype=torch.float32)
            path = os.path.join(d, "model.safetensors")
            f = SafetensorsFile(path)
            state = {k: f.get(k).clone() for k in f.keys()}
            f.close()
            if "lm_head.weight" not in state:
                state["lm_head.weight"] = state["model.embed_tokens.weight"].clone()
                save_safetensors(path, state)
            with open(os.path.join(d, "config.json")) as fh:
                c = json.load(fh)
            if not isinstance(c.get("eos_token_id"), int):   # the reference reads one integer or null
                c["eos_token_id"] = None
            with open(os.path.join(d, "config.json"), "w") as fh:
                json.dump(c, fh)
            raw = os.path.join(d, "logits.f32")
            res = subprocess.run([driver, "logits", "--model", d, "--tokens", ",".join(map(str, PROMPTS[name])),
                                  "--decode", str(DECODE), "--out", raw], capture_output=True, text=True)
            if res.returncode != 0:
                raise SystemExit(f"ref_driver failed on tiny {name}: {res.stderr}")
            ids = json.loads(res.stdout.strip().splitlines()[-1])["ids"]
            logits = np.fromfile(raw, dtype="<f4").reshape(DECODE + 1, cfg.vocab_size)
        out[f"{name}.logits"] = torch.from_numpy(logits.copy())
        out[f"{name}.prompt"] = torch.tensor(PROMPTS[name], dtype=torch.int32)
        out[f"{name}.ids"] = torch.tensor(ids, dtype=torch.int32)
        meta[name] = f"seed {seed}"
        print(f"tiny {name}: reference chose {ids}")
    save_safetensors(os.path.join(HERE, "reference_logits.safetensors"), out,
                     metadata={"source": "zscey/tiny-llm engine, unmodified, through baseline/ref_driver.cpp", **meta})
    print("wrote tests/golden/reference_logits.safetensors")


if __name__ == "__main__":
    main()
