"""Checks the parts of tests/plain_llama.py against the golden tensors that zscey/tiny-llm ships
for its own kernel tests, and writes the largest differences to tests/golden/plain_vs_reference.json.

tiny-llm's model code is CUDA only and cannot be built or imported on a CPU, so this is the
anchor the plain implementation has: the inputs are rebuilt here from the recipes in tiny-llm's
tests (ramps such as (i % 100) / 100), the expected outputs are read from its
tests/datas/*.safetensors, and every part of the plain implementation that has a golden tensor
is compared with it.

Usage:  python tests/golden/make_golden.py /path/to/tiny-llm
"""
import json
import os
import sys

import torch
from safetensors import safe_open

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import plain_llama as pl  # noqa: E402


def golden(ref_root, name, key="res"):
    with safe_open(os.path.join(ref_root, "tests", "datas", name), "pt") as f:
        return f.get_tensor(key)


def ramp(n, shift=0, div=100.0):
    i = torch.arange(n, dtype=torch.int64) + shift
    return (i % 100).to(torch.float32) / div


def check_rms_norm(ref_root):
    # tests/ops/cuda/test_norm.cpp:8-47
    b, l, d = 2, 107, 241
    x = ramp(b * l * d).view(b, l, d)
    w = ramp(d)
    got = pl.rms_norm(x, w, 1.192e-7)
    return float((got - golden(ref_root, "rms_norm_b2l107d241.safetensors")).abs().max())


def check_rope_tables(ref_root):
    # tests/ops/cuda/test_rope.cpp:8-39: the golden holds each half twice
    cos, sin = pl.rope_tables(2, 96, 10000.0)
    gc = golden(ref_root, "rope_s2_d96.safetensors", "cos")[0]
    gs = golden(ref_root, "rope_s2_d96.safetensors", "sin")[0]
    d = max(float((cos - gc[:, :48]).abs().max()), float((cos - gc[:, 48:]).abs().max()),
            float((sin - gs[:, :48]).abs().max()), float((sin - gs[:, 48:]).abs().max()))
    return d


def check_apply_rope(ref_root):
    # tests/ops/cuda/test_rope.cpp:41-98
    b, h, q, d, qs, qe = 3, 4, 2, 96, 1, 5
    cos, sin = pl.rope_tables(2, d, 10000.0)
    x = torch.ones(b, h, qe, d)
    x[:, :, qs:qs + q, :] = ramp(b * h * q * d).view(b, h, q, d)
    pos = torch.tensor([0, 1] * b).view(b, q)
    out = x.clone()
    for bi in range(b):
        rows = x[bi, :, qs:qs + q, :].permute(1, 0, 2)  # [q, h, d]
        out[bi, :, qs:qs + q, :] = pl.apply_rope(rows, cos, sin, pos[bi]).permute(1, 0, 2)
    g = golden(ref_root, "apply_rope_b3_h4_q2_d96_qs1qe5.safetensors")
    return float((out - g).abs().max())


def attention_inputs(batch, nq, nkv, ql, kl, d):
    q = ramp(batch * nq * ql * d).view(batch, nq, ql, d)
    k = ramp(batch * nkv * kl * d, shift=1).view(batch, nkv, kl, d)
    v = ramp(batch * nkv * kl * d, shift=2).view(batch, nkv, kl, d)
    return q, k, v


def check_attention(ref_root, causal):
    # tests/ops/cuda/test_flash_attention.cpp:8-90 (no mask), 92-170 (causal)
    batch, nq, nkv, ql, d = 2, 4, 2, 107, 61
    kl = ql if causal else 123
    q, k, v = attention_inputs(batch, nq, nkv, ql, kl, d)
    name = "causal_attn_res_b2l107q4k2d61.safetensors" if causal else "attn_res_b2q107h4k123h2d61.safetensors"
    g = golden(ref_root, name).reshape(-1)
    outs = []
    for bi in range(batch):
        o = pl.attention(q[bi].permute(1, 0, 2), k[bi].permute(1, 0, 2), v[bi].permute(1, 0, 2),
                         torch.arange(ql), causal=causal)  # [ql, nq, d]
        outs.append(o)
    o = torch.stack(outs)  # [b, ql, nq, d] = the kernel's [batch, q_length, q_head*dim]
    d1 = float((o.reshape(-1) - g).abs().max())
    d2 = float((o.permute(0, 2, 1, 3).reshape(-1) - g).abs().max())
    return min(d1, d2)


def check_attention_block(ref_root):
    # tests/runtime/cuda/test_attention_runtime.cpp:163-318: one attention block at TinyLlama
    # sizes, 3 prompt tokens then 2 decoded ones; as whole-sequence math that is 5 causal rows.
    hidden, nq, nkv, hd = 2048, 32, 4, 64
    w_qo = ramp(hidden * hidden, div=10000.0).view(hidden, hidden)
    w_kv = ramp(nkv * hd * hidden, div=10000.0).view(nkv * hd, hidden)
    w = {"q_proj.weight": w_qo, "o_proj.weight": w_qo, "k_proj.weight": w_kv, "v_proj.weight": w_kv}
    x = ramp(5 * hidden, div=10000.0).view(5, hidden)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "hidden_size": hidden}
    gc = golden(ref_root, "llama_attn_res_b1q5h2048.safetensors", "cos")[0]
    gs = golden(ref_root, "llama_attn_res_b1q5h2048.safetensors", "sin")[0]
    cos, sin = pl.rope_tables(5, hd, 10000.0)
    table_diff = max(float((cos - gc).abs().max()), float((sin - gs).abs().max()))
    out = pl.attention_block(x, w, "", cfg, cos, sin, torch.arange(5))
    g = golden(ref_root, "llama_attn_res_b1q5h2048.safetensors")[0]
    return float((out - g).abs().max()), table_diff, float(g.abs().max())


def iramp(n):
    return (torch.arange(n, dtype=torch.int64) % 100).to(torch.float32)


def check_gemm(ref_root):
    # tests/ops/cuda/test_gemm.cpp:160-199: C = A W^T with integer ramps (every sum is exact in 32-bit)
    m, d, n = 127, 255, 353
    out = pl.linear(iramp(m * d).view(m, d), iramp(n * d).view(n, d))
    return float((out - golden(ref_root, "gemm_m127d255n353.safetensors").view(m, n)).abs().max())


def check_gemm_to_heads(ref_root):
    # tests/ops/cuda/test_gemm.cpp:201-260: the projection whose result goes head-major into rows
    # [q_start, q_start + q) of a [b, heads, q_end, dim] buffer that held ones (the reference's Q projection)
    b, q, d, heads, dim, q_start = 2, 61, 255, 4, 88, 3
    q_end = q_start + q + 13
    y = pl.linear(iramp(b * q * d).view(b, q, d), iramp(heads * dim * d).view(heads * dim, d))   # [b, q, heads * dim]
    dst = torch.ones(b, heads, q_end, dim)
    dst[:, :, q_start:q_start + q, :] = y.view(b, q, heads, dim).permute(0, 2, 1, 3)
    g = golden(ref_root, "gemm_b2q61d255oh4od88qs3qe77.safetensors").view(b, heads, q_end, dim)
    return float((dst - g).abs().max())


def check_gemm_from_heads(ref_root):
    # tests/ops/cuda/test_gemm.cpp:262-306: head-major [b, heads, q, d] rows joined per token, then the
    # product (the reference's output projection)
    b, h, q, d, out_d = 2, 4, 127, 61, 313
    x = iramp(b * h * q * d).view(b, h, q, d).permute(0, 2, 1, 3).reshape(b, q, h * d)
    out = pl.linear(x, iramp(out_d * h * d).view(out_d, h * d))
    return float((out - golden(ref_root, "gemm_b2h4q127d61od313.safetensors").view(b, q, out_d)).abs().max())


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")
    block, table, scale = check_attention_block(ref_root)
    result = {
        "rms_norm_b2l107d241": check_rms_norm(ref_root),
        "rope_s2_d96_tables": check_rope_tables(ref_root),
        "apply_rope_b3_h4_q2_d96": check_apply_rope(ref_root),
        "attn_nomask_b2q107h4k123h2d61": check_attention(ref_root, False),
        "attn_causal_b2l107q4k2d61": check_attention(ref_root, True),
        "gemm_m127d255n353": check_gemm(ref_root),
        "gemm_to_heads_b2q61d255oh4od88qs3qe77": check_gemm_to_heads(ref_root),
        "gemm_from_heads_b2h4q127d61od313": check_gemm_from_heads(ref_root),
        "llama_attn_block_b1q5h2048": block,
        "llama_attn_block_tables": table,
        "llama_attn_block_max_abs_of_golden": scale,
    }
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_vs_reference.json")
    with open(out, "w") as f:
        json.dump({"what": "max |plain - tiny-llm golden| per part, float32", "max_abs_diff": result}, f, indent=1)
        f.write("\n")
    print(json.dumps(result, indent=1))


if __name__ == "__main__":
    main()
