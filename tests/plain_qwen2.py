"""A plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache, no
paging, no batching, one function per part.  It is the oracle of the tests and shares no
code with the package: it reads ``config.json`` and the safetensors file itself (through
the ``safetensors`` package) and works on checkpoint tensor names.

Every function restates a formula of the reference (ashwinsreedhar28/emberserve; paths
are inside that project) and cites it.  ``tests/golden/`` holds logits that the
reference's own model code produced on the CPU for two tiny random models; the test
``test_plain_vs_reference_golden`` ties this file to them.

Arithmetic runs in `dtype` (float64 by default, so that it is the "true" answer that both
the 32-bit and the bfloat16 engine are compared with); rotary angles are formed in
float32 exactly as the reference forms them, because the angle at a far position depends
on the rounding of ``inv_freq``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ---- reading a model folder (independent of the package's loader) ----------------------

def read_model_dir(model_dir) -> tuple[dict, dict[str, torch.Tensor]]:
    from safetensors import safe_open

    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    weights: dict[str, torch.Tensor] = {}
    for path in sorted(Path(model_dir).glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for key in f.keys():
                weights[key] = f.get_tensor(key)
    return cfg, weights


def geometry(cfg: dict) -> dict:
    """Sizes and constants from config.json; defaults as emberserve/config.py:202-234."""
    heads = cfg["num_attention_heads"]
    window = cfg.get("sliding_window")
    if window in (None, 0) or not cfg.get("use_sliding_window", True):
        window = None
    layers = cfg["num_hidden_layers"]
    return dict(
        layers=layers, hidden=cfg["hidden_size"], heads=heads,
        kv_heads=cfg.get("num_key_value_heads") or heads,
        head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
        inter=cfg["intermediate_size"], vocab=cfg["vocab_size"],
        eps=cfg.get("rms_norm_eps", 1e-6), theta=cfg.get("rope_theta", 1_000_000.0),
        tied=cfg.get("tie_word_embeddings", True), bias=cfg.get("attention_bias", True),
        window=window, max_window_layers=cfg.get("max_window_layers", layers) if window else 0)


# ---- the parts ------------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """h0[n] = E[ids[n]]  (emberserve/model/qwen2.py:172,182)."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """weight * (x * rsqrt(mean(x^2, -1) + eps))  (emberserve/model/ops.py:51-55)."""
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """float32 angles [T, D]: inv_freq = 1 / theta^(2i/D); freqs = pos (x) inv_freq;
    emb = cat(freqs, freqs)  (emberserve/model/rope.py:68-82)."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (float(theta) ** exponent)
    freqs = torch.outer(positions.to(torch.float32), inv_freq.to(positions.device))
    return torch.cat((freqs, freqs), dim=-1)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(x1, x2) -> (-x2, x1) over the halves of the last dim (emberserve/model/rope.py:19-23)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, D]; x*cos + rotate_half(x)*sin  (emberserve/model/ops.py:66-81)."""
    c = angles.to(x.dtype).cos()[:, None, :]
    s = angles.to(x.dtype).sin()[:, None, :]
    return x * c + rotate_half(x) * s


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: int | None = None) -> torch.Tensor:
    """q: [T, H, D], k/v: [T, Hkv, D] of ONE whole sequence.  Query head h reads KV head
    h // (H/Hkv); scores = q.k / sqrt(D); key j is hidden from query i iff j > i; softmax
    over keys; out = P.V  (emberserve/attn/base.py:105-128).  With a window of W keys, key
    j is also hidden iff j <= i - W."""
    t, h, d = q.shape
    groups = h // k.shape[1]
    qf = q.transpose(0, 1)                                   # [H, T, D]
    kf = k.repeat_interleave(groups, dim=1).transpose(0, 1)  # [H, T, D]
    vf = v.repeat_interleave(groups, dim=1).transpose(0, 1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) / math.sqrt(d)
    i = torch.arange(t, device=q.device)[:, None]
    j = torch.arange(t, device=q.device)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, vf).transpose(0, 1)           # [T, H, D]


def attention_block(x: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, g: dict,
                    positions: torch.Tensor, window: int | None) -> torch.Tensor:
    """q/k/v projections with bias, rotary on q and k, attention, output projection without
    bias (emberserve/model/qwen2.py:88-114)."""
    t = x.shape[0]

    def proj(name: str) -> torch.Tensor:
        y = x @ w[f"{prefix}.{name}.weight"].T
        if g["bias"]:
            y = y + w[f"{prefix}.{name}.bias"]
        return y

    q = proj("q_proj").view(t, g["heads"], g["head_dim"])
    k = proj("k_proj").view(t, g["kv_heads"], g["head_dim"])
    v = proj("v_proj").view(t, g["kv_heads"], g["head_dim"])
    angles = rope_angles(positions, g["head_dim"], g["theta"])
    q, k = apply_rope(q, angles), apply_rope(k, angles)
    out = causal_attention(q, k, v, window)
    return out.reshape(t, g["heads"] * g["head_dim"]) @ w[f"{prefix}.o_proj.weight"].T


def swiglu(x: torch.Tensor, w: dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x))  (emberserve/model/qwen2.py:53-61, ops.py:84-87)."""
    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    return (torch.nn.functional.silu(gate) * up) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(h: torch.Tensor, w: dict[str, torch.Tensor], i: int, g: dict,
                  positions: torch.Tensor) -> torch.Tensor:
    """h += attn(norm1(h)); h += mlp(norm2(h))  (emberserve/model/qwen2.py:122-164)."""
    p = f"model.layers.{i}"
    window = g["window"] if (g["window"] is not None and i >= g["max_window_layers"]) else None
    h = h + attention_block(rms_norm(h, w[f"{p}.input_layernorm.weight"], g["eps"]), w,
                            f"{p}.self_attn", g, positions, window)
    h = h + swiglu(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], g["eps"]), w, f"{p}.mlp")
    return h


def forward_logits(cfg: dict, weights: dict[str, torch.Tensor], token_ids: list[int],
                   dtype: torch.dtype = torch.float64, device: str = "cpu") -> torch.Tensor:
    """Logits [T, vocab] of every position of one whole sequence
    (emberserve/model/qwen2.py:180-187,214-230).  `device`: where the same plain arithmetic
    runs (sequences of thousands of tokens need more memory than a host may have)."""
    g = geometry(cfg)
    w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}
    ids = torch.tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(len(token_ids), device=device)
    h = embedding(w["model.embed_tokens.weight"], ids)
    for i in range(g["layers"]):
        h = decoder_layer(h, w, i, g, positions)
    h = rms_norm(h, w["model.norm.weight"], g["eps"])
    head = w["model.embed_tokens.weight"] if g["tied"] else w["lm_head.weight"]
    return h @ head.T


def greedy_generate(cfg: dict, weights: dict[str, torch.Tensor], prompt: list[int],
                    max_tokens: int, dtype: torch.dtype = torch.float64) -> list[int]:
    """Greedy continuation by recomputing the whole sequence for every token."""
    ids = list(prompt)
    out: list[int] = []
    for _ in range(max_tokens):
        nxt = int(torch.argmax(forward_logits(cfg, weights, ids, dtype)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out
