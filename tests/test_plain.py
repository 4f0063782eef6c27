"""The plain implementation against the reference's own model code (golden logits made by
tests/golden/make_golden.py), and its parts against independent restatements."""

from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from tiny_configs import ALL, SEEDS

from emberserve_b200.registry import build_decoder
from emberserve_b200.weights.loader import random_checkpoint
from emberserve_b200.weights.safetensors_io import SafetensorsFile

GOLDEN = Path(__file__).resolve().parent / "golden"


def _checksum(tensors):
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_vs_reference_golden(name):
    meta = json.loads((GOLDEN / "golden.json").read_text())[name]
    cfg = ALL[name]
    # the very weights that went through the reference's model (stored beside its logits): the
    # anchor does not depend on what this torch draws from the seed
    stored = SafetensorsFile(GOLDEN / f"{name}_weights.safetensors")
    tensors = {n: stored.get(n).clone() for n in stored.names()}
    assert _checksum(tensors) == meta["weights_sha256"]
    assert set(tensors) == set(random_checkpoint(build_decoder(cfg), SEEDS[name], store_dtype=torch.float32))
    want = torch.from_numpy(np.load(GOLDEN / f"{name}_logits.npy")).double()
    got = plain.forward_logits(cfg.to_dict(), tensors, meta["tokens"], torch.float64)
    assert got.shape == want.shape
    assert float((got - want).abs().max()) <= 2e-6 * float(want.abs().max()) + 1e-6
    got32 = plain.forward_logits(cfg.to_dict(), tensors, meta["tokens"], torch.float32)
    assert float((got32.double() - want).abs().max()) <= 1e-5


def test_rope_against_complex_rotation():
    """Rotate-half rotary equals multiplication by exp(i*angle) of the pairs (x[i], x[i+D/2])."""
    torch.manual_seed(0)
    t, h, d, theta = 9, 3, 16, 10000.0
    x = torch.randn(t, h, d, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 5, 9, 33, 100, 101, 127])
    out = plain.apply_rope(x, plain.rope_angles(pos, d, theta))
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.outer(pos.float(), inv).double()
    z = torch.complex(x[..., :d // 2], x[..., d // 2:]) * torch.polar(torch.ones_like(ang), ang)[:, None, :]
    assert torch.allclose(out[..., :d // 2], z.real, atol=1e-12)
    assert torch.allclose(out[..., d // 2:], z.imag, atol=1e-12)
    assert torch.allclose(out[0], x[0])  # position 0 is the identity
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1))


def test_attention_loops():
    """causal_attention against explicit loops over heads, queries and keys."""
    torch.manual_seed(1)
    t, h, hkv, d, window = 11, 6, 2, 8, 4
    q, k, v = (torch.randn(t, n, d, dtype=torch.float64) for n in (h, hkv, hkv))
    for w in (None, window):
        got = plain.causal_attention(q, k, v, w)
        for head in range(h):
            kv = head // (h // hkv)
            for i in range(t):
                lo = 0 if w is None else max(0, i - w + 1)
                s = torch.tensor([float(q[i, head] @ k[j, kv]) / math.sqrt(d) for j in range(lo, i + 1)],
                                 dtype=torch.float64)
                p = torch.softmax(s, 0)
                want = sum(p[j - lo] * v[j, kv] for j in range(lo, i + 1))
                assert torch.allclose(got[i, head], want, atol=1e-12)


def test_rms_norm_and_swiglu():
    torch.manual_seed(2)
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.randn(12, dtype=torch.float64)
    want = torch.stack([w * row / math.sqrt(float((row * row).sum()) / 12 + 1e-5) for row in x])
    assert torch.allclose(plain.rms_norm(x, w, 1e-5), want, atol=1e-12)
    ws = {"m.gate_proj.weight": torch.randn(7, 12, dtype=torch.float64),
          "m.up_proj.weight": torch.randn(7, 12, dtype=torch.float64),
          "m.down_proj.weight": torch.randn(12, 7, dtype=torch.float64)}
    g, u = x @ ws["m.gate_proj.weight"].T, x @ ws["m.up_proj.weight"].T
    want = (g / (1 + torch.exp(-g)) * u) @ ws["m.down_proj.weight"].T
    assert torch.allclose(plain.swiglu(x, ws, "m"), want, atol=1e-12)


def test_window_changes_only_far_positions():
    cfg = ALL["tiny_c"]
    tensors = random_checkpoint(build_decoder(cfg), SEEDS["tiny_c"], store_dtype=torch.float32)
    ids = list(range(3, 3 + 40))
    with_w = plain.forward_logits(cfg.to_dict(), tensors, ids)
    without = plain.forward_logits(cfg.replace(sliding_window=None, max_window_layers=0).to_dict(), tensors, ids)
    w = cfg.sliding_window
    assert torch.allclose(with_w[:w], without[:w], atol=1e-12)
    assert float((with_w[w:] - without[w:]).abs().max()) > 1e-6
