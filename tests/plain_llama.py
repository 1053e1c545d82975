"""Plain, slow Llama decoder for the tests: whole sequences, no cache, one function per part.

It is written from the formulas of zscey/tiny-llm's kernels and parser (each function cites the
file and lines it restates) and shares no code with the `tiny_llm_b200` package: it reads
`config.json` with `json` and the weights with the `safetensors` library, and computes with
plain torch tensor arithmetic on the CPU.

tiny-llm's model math exists only as CUDA kernels (it has no CPU forward pass), so it cannot be
imported or compiled into a CPU oracle.  Two anchors tie this file to it all the same:
`tests/golden/make_golden.py` checks its parts against the golden tensors that tiny-llm ships for its
own kernel tests (tests/datas/*.safetensors), and `tests/golden/reference_logits.safetensors` holds
whole-model logits that tiny-llm's own engine computed on a B200 (prompt whole, then token by token,
paged mode) for the tiny test configurations; tests/test_plain.py compares `forward` with them.

`quant` is the storage rounding of the path that is being checked: the identity for the 32-bit
path; for the bfloat16 path a round-trip through bfloat16 at the places where that path stores
bfloat16 (projection outputs, attention output, activations), while statistics, softmax,
rotation and the residual stream stay in 32-bit.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

Quant = Callable[[torch.Tensor], torch.Tensor]


def no_quant(x: torch.Tensor) -> torch.Tensor:
    return x


def bf16_quant(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


# ----------------------------------------------------------------------------- loading


def load_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def load_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), "pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(dtype)
    return out


# ----------------------------------------------------------------------------- parts


def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x[t,:] = W_e[token[t],:]  (tiny_llm/ops/cuda/embedding.cu:10-29)."""
    return table[tokens.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y_j = (w_j * x_j) / sqrt(sum_j(x_j^2 / H) + eps): weight first, eps inside the root
    (tiny_llm/ops/cuda/norm.cu:29-48)."""
    h = x.shape[-1]
    ms = (x * x / h).sum(dim=-1, keepdim=True)
    return (weight * x) / torch.sqrt(ms + eps)


def rope_tables(max_len: int, head_dim: int, theta: float):
    """ang[p,i] = p * theta^(-i/(hd/2)), i in [0, hd/2), in 64-bit; stored as 32-bit cos and sin
    (tiny_llm/ops/cuda/rope.cu:12-24)."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    p = torch.arange(max_len, dtype=torch.float64)
    ang = p[:, None] * torch.pow(torch.tensor(theta, dtype=torch.float64), -i / half)[None, :]
    return torch.cos(ang).float(), torch.sin(ang).float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor):
    """Rotate-half pairing (i, i+hd/2): x'_i = c x_i - s x_{i+hd/2}; x'_{i+hd/2} = s x_i + c x_{i+hd/2}
    (tiny_llm/ops/cuda/rope.cu:26-56).  x: [T, heads, hd]."""
    half = x.shape[-1] // 2
    c = cos[positions.long()][:, None, :].to(x.dtype)
    s = sin[positions.long()][:, None, :].to(x.dtype)
    re, im = x[..., :half], x[..., half:]
    return torch.cat([c * re - s * im, s * re + c * im], dim=-1)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """C[m,n] = sum_d A[m,d] W[n,d]; weights are row-major [out, in], no bias
    (tiny_llm/ops/cuda/gemm.cu:67-106)."""
    return x @ w.t()


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor,
              window: Optional[int] = None, causal: bool = True, quant: Quant = no_quant) -> torch.Tensor:
    """Scaled dot-product attention with grouped heads, full softmax (the reference's running
    softmax over 64-key tiles is the same function; tiny_llm/ops/cuda/flash_attention.cu:50-117,
    338-442).  q: [Tq, nq, hd]; k, v: [Tk, nkv, hd]; q head h reads kv head h // (nq/nkv); scores are
    (q / sqrt(hd)) . k; key j is visible to the query at absolute position p iff j <= p (and
    j > p - window if a window is given).  The reference compares a chunk-local query index with
    the absolute key index (flash_attention.cu:63-66, 402-405), which is the same rule when the
    chunk starts at position 0, the only case it runs; the absolute rule is used here.
    `quant` rounds the unnormalised probabilities exp(s - max) where they enter the P.V product (the
    bfloat16 path feeds them to the tensor cores in bfloat16); their sum stays 32-bit."""
    tq, nq, hd = q.shape
    tk, nkv, _ = k.shape
    group = nq // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    kj = torch.arange(tk)
    if causal:
        visible = kj[None, :] <= q_pos.long()[:, None]
        if window is not None:
            visible &= kj[None, :] > (q_pos.long()[:, None] - window)
    else:
        visible = torch.ones(tq, tk, dtype=torch.bool)
    for h in range(nq):
        s = (q[:, h, :] * scale) @ k[:, h // group, :].t()
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        out[:, h, :] = (quant(p) @ v[:, h // group, :]) / p.sum(dim=-1, keepdim=True)
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x))  (tiny_llm/ops/cuda/silu.cu:7-12)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(y: torch.Tensor, wg, wu, wd, quant: Quant = no_quant) -> torch.Tensor:
    """m = (silu(y Wg^T) * (y Wu^T)) Wd^T  (tiny_llm/parser/llama_parser.cpp:225-249;
    product: tiny_llm/ops/cuda/arithmetic.cu:7-22)."""
    z = quant(silu(linear(y, wg)) * linear(y, wu))
    return linear(z, wd)


def attention_block(h, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, cos, sin, positions,
                    quant: Quant = no_quant, window: Optional[int] = None) -> torch.Tensor:
    """Q/K/V projections, RoPE on Q and K, attention, output projection
    (tiny_llm/runtime/cuda/cuda_kernels.cpp:336-385)."""
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nq
    t = h.shape[0]
    q = quant(linear(h, w[prefix + "q_proj.weight"])).view(t, nq, hd)
    k = quant(linear(h, w[prefix + "k_proj.weight"])).view(t, nkv, hd)
    v = quant(linear(h, w[prefix + "v_proj.weight"])).view(t, nkv, hd)
    q = quant(apply_rope(q, cos, sin, positions))
    k = quant(apply_rope(k, cos, sin, positions))
    o = quant(attention(q, k, v, positions, window=window, quant=quant)).reshape(t, nq * hd)
    return linear(o, w[prefix + "o_proj.weight"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], quant: Quant = no_quant,
            dtype=torch.float32, rows: Optional[List[int]] = None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence starting at position 0: embedding, then per layer
    norm -> attention -> residual -> norm -> SwiGLU -> residual, final norm, LM head
    (tiny_llm/parser/llama_parser.cpp:164-276).  The residual stream is never rounded.
    `rows`: the positions whose logits are wanted ([len(rows), V]; the reference itself takes the
    last row only, tiny_llm/ops/cuda/gemm_q1_helper.cu:99-124); None: all."""
    w = {k: v.to(dtype) for k, v in w.items()}
    toks = torch.tensor(tokens, dtype=torch.long)
    t = toks.numel()
    positions = torch.arange(t)
    nq = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nq
    eps = cfg["rms_norm_eps"]
    cos, sin = rope_tables(cfg["max_position_embeddings"], hd, cfg.get("rope_theta", 10000.0))
    x = embedding(w["model.embed_tokens.weight"], toks)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = quant(rms_norm(x, w[p + "input_layernorm.weight"], eps))
        x = x + attention_block(h, w, p + "self_attn.", cfg, cos, sin, positions, quant)
        h = quant(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
        x = x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"], quant)
    if rows is not None:
        x = x[torch.tensor(rows, dtype=torch.long)]
    x = quant(rms_norm(x, w["model.norm.weight"], eps))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(x, head)


# ----------------------------------------------------------------------------- sampling


def greedy(logits: torch.Tensor) -> int:
    """First maximum: strict '>' keeps the lowest index on ties
    (tiny_llm/logit_processors/argmax_processor.cpp:24-31)."""
    best = 0
    for j in range(1, logits.numel()):
        if logits[j] > logits[best]:
            best = j
    return best


def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """Temperature -> top-k -> top-p, the reference's chain (tiny_llm/pipeline/pipeline.cpp:157-161).
    Returns (kept token ids in ascending order, their probabilities).
    temperature: logits / T (temperature_processor.hpp:12-19).
    top-k: keep the k largest (sort_processors.cpp:53-78); k == 0 or k >= V keeps all here.
    top-p: sort descending, softmax over the kept ones, drop from the tail while the dropped mass
    stays <= 1 - p, keep at least one (sort_processors.cpp:107-142)."""
    x = logits.double() / temperature
    v = x.numel()
    order = torch.argsort(x, descending=True, stable=True)
    if 0 < top_k < v:
        order = order[:top_k]
    xs = x[order]
    p = torch.exp(xs - xs[0])
    p = p / p.sum()
    if top_p < 1.0:
        remain = 1.0 - top_p
        idx = len(order) - 1
        while idx >= 1:
            remain -= float(p[idx])
            if remain < 0:
                break
            idx -= 1
        order = order[: idx + 1]
        xs = x[order]
    p = torch.exp(xs - xs.max())
    p = p / p.sum()
    ids, perm = torch.sort(order)
    return ids, p[perm]


def multinomial(ids: torch.Tensor, probs: torch.Tensor, u: float) -> int:
    """Inverse CDF over the kept tokens with u in [0,1): subtract probabilities until negative
    (tiny_llm/logit_processors/sample_processors.cpp:40-48); the kept tokens are walked in
    ascending token id."""
    r = u
    for i in range(len(ids)):
        r -= float(probs[i])
        if r < 0:
            return int(ids[i])
    return int(ids[-1])
