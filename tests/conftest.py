import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# Two tiny configurations that differ in every size and option, and a third with a head size that
# is not hidden/heads and an odd vocabulary.  initializer_range is larger than 0.02 so that attention
# is peaked and a wrong or missing key moves the logits far beyond rounding.
TINY_A = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, intermediate_size=176, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=128, tie_word_embeddings=False,
              hidden_act="silu", attention_bias=False, rope_scaling=None, initializer_range=0.15,
              eos_token_id=2, torch_dtype="float32")
TINY_B = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=3, num_key_value_heads=1, intermediate_size=256, vocab_size=384,
              rope_theta=500000.0, rms_norm_eps=1e-6, max_position_embeddings=256, tie_word_embeddings=True,
              hidden_act="silu", attention_bias=False, rope_scaling=None, initializer_range=0.12,
              eos_token_id=[5, 7], torch_dtype="float32")
TINY_C = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=1, hidden_size=80,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=208, vocab_size=331,
              rope_theta=1000.0, rms_norm_eps=1e-4, max_position_embeddings=192, tie_word_embeddings=False,
              hidden_act="silu", initializer_range=0.1, torch_dtype="float32")
TINY = {"A": (TINY_A, 16, 0), "B": (TINY_B, 8, 1), "C": (TINY_C, 32, 2)}  # config, page size, seed


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations with random weights, made once per session."""
    import torch

    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.weights import write_random_model

    out = {}
    for name, (cfg, _page, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(str(d), LlamaConfig.from_dict(cfg), seed=seed, dtype=torch.float32)
        out[name] = str(d)
    return out
