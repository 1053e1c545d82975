"""The plain implementation itself (no GPU): against tiny-llm's golden tensors where the checkout
is at hand, and against independent restatements."""
import json
import math
import os

import pytest
import torch

import plain_llama as pl
from conftest import TINY_A, TINY_B

REF = os.environ.get("TINY_LLM_REFERENCE", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))   # a tiny-llm checkout, if one lies beside the repository


def test_committed_golden_differences_are_small():
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "golden", "plain_vs_reference.json")) as f:
        d = json.load(f)["max_abs_diff"]
    assert all(v < 1e-6 for k, v in d.items() if not k.endswith("max_abs_of_golden")), d


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "datas")), reason="tiny-llm checkout not at hand")
def test_parts_match_the_reference_golden_tensors():
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_golden as mg
    assert mg.check_rms_norm(REF) < 1e-5            # the reference's own tolerances (test_norm.cpp:45)
    assert mg.check_rope_tables(REF) < 1e-6
    assert mg.check_apply_rope(REF) < 1e-4          # test_rope.cpp:89
    assert mg.check_attention(REF, False) < 1e-5    # test_flash_attention.cpp:87
    assert mg.check_attention(REF, True) < 1e-5
    assert mg.check_attention_block(REF)[0] < 1e-5  # test_attention_runtime.cpp:248


def test_attention_against_a_per_query_loop():
    torch.manual_seed(0)
    tq, nq, nkv, hd = 9, 4, 2, 16
    q, k, v = torch.randn(tq, nq, hd), torch.randn(tq, nkv, hd), torch.randn(tq, nkv, hd)
    pos = torch.arange(tq)
    for window in (None, 3):
        got = pl.attention(q, k, v, pos, window=window)
        for t in range(tq):
            lo = 0 if window is None else max(0, t - window + 1)
            for h in range(nq):
                s = torch.tensor([float(q[t, h] @ k[j, h // 2]) / math.sqrt(hd) for j in range(lo, t + 1)])
                p = torch.softmax(s, 0)
                want = sum(p[i] * v[lo + i, h // 2] for i in range(len(p)))
                assert torch.allclose(got[t, h], want, atol=1e-5)


def test_causality_and_double_precision_agreement(model_dirs):
    for name, cfg in (("A", TINY_A), ("B", TINY_B)):
        c, w = pl.load_config(model_dirs[name]), pl.load_weights(model_dirs[name])
        toks = list(range(3, 40))
        full = pl.forward(c, w, toks)
        part = pl.forward(c, w, toks[:17])
        assert torch.allclose(full[:17], part, atol=1e-5)            # later tokens do not reach back
        dbl = pl.forward(c, w, toks, dtype=torch.float64)
        assert float((full.double() - dbl).abs().max()) < 1e-4
        assert full.shape == (37, cfg["vocab_size"])


def test_sampling_chain():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0, 0.5])
    assert pl.greedy(logits) == 1                                   # first maximum
    ids, p = pl.sampling_distribution(logits, 1.0, 0, 1.0)
    assert ids.tolist() == [0, 1, 2, 3, 4, 5] and abs(float(p.sum()) - 1) < 1e-12
    ids, p = pl.sampling_distribution(logits, 0.5, 3, 1.0)
    assert ids.tolist() == [1, 2, 3]                                # the three largest
    assert torch.allclose(p, torch.softmax(torch.tensor([6.0, 4.0, 6.0]).double(), 0))
    ids, p = pl.sampling_distribution(logits, 1.0, 0, 0.6)
    assert ids.tolist() == [1, 3]                                   # the tail is dropped while its mass <= 0.4
    ids, _ = pl.sampling_distribution(logits, 1.0, 0, 0.0)
    assert ids.tolist() == [1]                                      # at least one token stays
    assert pl.multinomial(torch.tensor([4, 7, 9]), torch.tensor([0.2, 0.5, 0.3]), 0.19) == 4
    assert pl.multinomial(torch.tensor([4, 7, 9]), torch.tensor([0.2, 0.5, 0.3]), 0.25) == 7
    assert pl.multinomial(torch.tensor([4, 7, 9]), torch.tensor([0.2, 0.5, 0.3]), 0.9999) == 9


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_model_against_the_logits_of_tiny_llm_itself(name, tmp_path):
    """tests/golden/reference_logits.safetensors holds what zscey/tiny-llm's own engine computes
    (unmodified, run on a B200 through baseline/ref_driver.cpp; made by tests/golden/make_reference_logits.py)
    for a short prompt run whole and six tokens decoded greedily one by one in paged mode, on the tiny
    configurations with the weights write_random_model makes.  The plain implementation, whole sequence and
    no cache, must give the same logits and choose the same ids: this pins the order of the parts
    (norm, attention, residual, norm, SwiGLU, residual, final norm, output matrix), which the goldens of
    single kernels cannot."""
    import os
    from conftest import TINY
    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.weights import SafetensorsFile, write_random_model
    gold = SafetensorsFile(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_logits.safetensors"))
    cfg_d, _page, seed = TINY[name]
    write_random_model(str(tmp_path), LlamaConfig.from_dict(cfg_d), seed=seed, dtype=torch.float32)
    cfg, w = pl.load_config(str(tmp_path)), pl.load_weights(str(tmp_path))
    prompt, ids, want = gold.get(f"{name}.prompt").tolist(), gold.get(f"{name}.ids").tolist(), gold.get(f"{name}.logits").clone()
    gold.close()
    logits = pl.forward(cfg, w, prompt + ids)
    rows = logits[len(prompt) - 1: len(prompt) - 1 + want.shape[0]]
    assert float((rows - want).abs().max()) <= 2e-5, float((rows - want).abs().max())
    assert [pl.greedy(r) for r in rows[:-1]] == ids
