"""Correctness at the context lengths that speeds are quoted for: 8 k, 16 k and 32 k keys.

Kernel level: the decode attention (the fused kernel and the unfused pair, with the split of
keys that the engine would pick, up to 64 blocks per KV head, window on and off), the tcgen05
prompt attention (a portion of 8,192 tokens; a portion of 2,048 tokens behind a cached prefix
of 30 k keys) and the rotary table up to position 32,768, each against a float64 restatement
over keys gathered from randomly permuted pages (the oracle style of the reference's
``tests/test_paged_attn.py:72-82``).  Inputs are peaked, and one case lets a single far key
(key 0 of a 32 k context) carry the whole result.  Engine level: one layer of the 7B
geometry, one request of about 9 k tokens, whole, with the tail decoded from CUDA graphs, and
in portions of 2,048 tokens, in bfloat16 against the plain implementation.  Every case holds
one layer and a few hundred MB at most.
"""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import kernel_refs as ref
import plain_qwen2 as plain
import replay_cases as rc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
BF16 = torch.bfloat16
TOL = dict(rtol=2e-2, atol=2e-2)


def K():
    from emberserve_b200 import kernels

    return kernels


def _pages(ctx_lens, ps, g, extra=7):
    """A block table whose rows own disjoint, randomly permuted pages of one pool."""
    width = max(-(-c // ps) for c in ctx_lens) + 1
    pages = len(ctx_lens) * width + extra
    table = torch.randperm(pages, device=DEV, generator=g)[: len(ctx_lens) * width].view(len(ctx_lens), width)
    return table.to(torch.int32), pages


# ---- the rotary table ---------------------------------------------------------------------------

@pytest.mark.parametrize("head_dim,theta", [(128, 1e6), (64, 1e6), (128, 1e4)])
def test_rope_table_to_position_32768(head_dim, theta):
    """cos and sin of float32(pos) * float32(inv_freq) in float32, as
    ``emberserve/model/rope.py:68-82`` forms them, for every position up to 32,768: the fastest
    pair turns about 5,000 times on the way, so a kernel that reduced the angle carelessly
    would show."""
    from emberserve_b200.parts.rope import inv_frequencies

    max_pos = 32768
    inv = inv_frequencies(head_dim, theta)
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    assert torch.equal(inv, 1.0 / (float(theta) ** exponent))  # the reference's inv_freq, bit for bit
    got = K().rope_table(inv.to(DEV), max_pos).cpu()
    freqs = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)  # float32 angles
    assert got.shape == (max_pos, head_dim // 2, 2)
    for part, fn in ((0, torch.cos), (1, torch.sin)):
        torch.testing.assert_close(got[..., part], fn(freqs), rtol=0, atol=2e-6)
        # and against the exact function of the same float32 angle
        torch.testing.assert_close(got[..., part].double(), fn(freqs.double()), rtol=0, atol=1e-6)


# ---- decode attention ---------------------------------------------------------------------------

def _decode_case(ctx, d, window, rotary, seed, nh=7, nkv=1, ps=16):
    """Rows whose contexts reach `ctx` keys and stop short of it at odd places; returns what the
    fused kernel, the unfused kernels and the float64 restatement make of the same inputs."""
    from emberserve_b200.parts.attention import decode_splits
    from emberserve_b200.parts.rope import inv_frequencies

    k = K()
    g = torch.Generator(device="cuda").manual_seed(seed)
    starts = [ctx - 1, ctx - 17, ctx // 2 + 3, 4097, 0, ctx - 128]
    b = len(starts)
    bt, pages = _pages([s + 1 for s in starts], ps, g)
    kc0 = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(BF16)
    vc0 = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(BF16)
    qkv0 = (torch.randn(b, (nh + 2 * nkv) * d, device=DEV, generator=g) * 3).to(BF16)  # peaked scores
    rot = d if rotary else 0
    table = k.rope_table(inv_frequencies(d, 1e6).to(DEV), ctx) if rotary else None
    cu = torch.arange(b + 1, device=DEV, dtype=torch.int32)
    st = torch.tensor(starts, device=DEV, dtype=torch.int32)
    rows = torch.arange(b, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(d)
    splits = decode_splits(b, nkv, ctx)

    def scratch():
        return torch.empty(max(1, k.attention_scratch_bytes(b, nh, d, splits) // 4), device=DEV)

    # the unfused pair: rotary + cache write, then attention over the cache
    qa, ka, va = qkv0.clone(), kc0.clone(), vc0.clone()
    k.rope_kv_write(qa, nh, nkv, d, st, rows, table, rot, ka, va, bt, ps)
    unfused = torch.full((b, nh * d), float("nan"), device=DEV, dtype=BF16)
    k.paged_attention(qa, unfused, ka, va, bt, cu, st, b, b, nh, nkv, d, scale, 1, window=window, splits=splits,
                      scratch=scratch())
    # the fused kernel on the raw projections
    kb, vb = kc0.clone(), vc0.clone()
    fused = torch.full((b, nh * d), float("nan"), device=DEV, dtype=BF16)
    k.decode_attention_fused(qkv0, fused, kb, vb, bt, cu, st, b, nh, nkv, d, scale, table, rot, True, window=window,
                             splits=splits, scratch=scratch())
    # the restatement, over the cache that the restated rotary kernel leaves
    qr, kr, vr = qkv0.clone(), kc0.clone(), vc0.clone()
    ref.rope_kv_write(qr, nh, nkv, d, st, rows, table, rot, kr, vr, bt, ps)
    want = torch.empty_like(unfused)
    ref.paged_attention(qr, want, kr, vr, bt, cu, st, b, b, nh, nkv, d, scale, 1, window=window,
                        compute_dtype=torch.float64)
    return splits, fused.float(), unfused.float(), want.float(), (kb, ka), (vb, va)


@pytest.mark.parametrize("ctx", [8192, 16384, 32768])
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("window", [None, 5000])
def test_decode_attention_at_long_contexts(ctx, d, window):
    splits, fused, unfused, want, keys, values = _decode_case(ctx, d, window, rotary=True, seed=ctx + d)
    assert splits >= 32, splits  # the split that the engine picks at this length: many blocks per KV head
    torch.testing.assert_close(unfused, want, **TOL)
    torch.testing.assert_close(fused, want, **TOL)
    assert torch.equal(keys[0], keys[1]) and torch.equal(values[0], values[1])


def test_decode_splits_reach_64_at_batch_1():
    from emberserve_b200.parts.attention import decode_splits

    assert decode_splits(1, 4, 32768, 148) == 64 and decode_splits(8, 4, 32768, 148) == 9
    assert decode_splits(1, 1, 8192, 148) == 64 and decode_splits(6, 1, 8192, 148) == 49


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("far", [0, 1, 16383, 32751])
def test_decode_far_key_of_a_32k_context_stands_out(d, far):
    """Batch 1, 32,767 cached keys, 64 blocks per KV head: head 0's query is made to point at one
    far key, so its output must be that key's value vector; a split that skipped its first tile,
    or a merge that lost a block, could not produce it."""
    k = K()
    nh, nkv, ps, ctx = 7, 1, 16, 32768
    g = torch.Generator(device="cuda").manual_seed(far + d)
    bt, pages = _pages([ctx], ps, g)
    kc = (torch.randn(pages, nkv, ps, d, device=DEV, generator=g) * 0.1).to(BF16)
    vc = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(BF16)
    qkv = torch.randn(1, (nh + 2 * nkv) * d, device=DEV, generator=g).to(BF16)
    page, slot = int(bt[0, far // ps]), far % ps
    kc[page, 0, slot] = (qkv[0, :d].float() * 50.0).to(BF16)
    cu = torch.tensor([0, 1], device=DEV, dtype=torch.int32)
    st = torch.tensor([ctx - 1], device=DEV, dtype=torch.int32)
    for fused in (False, True):
        for splits in (64, 37):
            scratch = torch.empty(k.attention_scratch_bytes(1, nh, d, splits) // 4, device=DEV)
            out = torch.full((1, nh * d), float("nan"), device=DEV, dtype=BF16)
            if fused:  # (no rotation, no write: the cache already holds the newest key)
                k.decode_attention_fused(qkv, out, kc, vc, bt, cu, st, 1, nh, nkv, d, 1.0, None, 0, False,
                                         splits=splits, scratch=scratch)
            else:
                k.paged_attention(qkv, out, kc, vc, bt, cu, st, 1, 1, nh, nkv, d, 1.0, 1, splits=splits,
                                  scratch=scratch)
            torch.testing.assert_close(out[0, :d].float(), vc[page, 0, slot].float(), **TOL)


# ---- prompt attention -----------------------------------------------------------------------------

def _prefill_case(q_len, start, d, window, seed, kernel, nh=7, nkv=1, ps=16, point_at=None):
    k = K()
    g = torch.Generator(device="cuda").manual_seed(seed)
    ctx = start + q_len
    bt, pages = _pages([ctx], ps, g)
    kc = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(BF16)
    vc = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(BF16)
    qkv = (torch.randn(q_len, (nh + 2 * nkv) * d, device=DEV, generator=g) * 3).to(BF16)
    if point_at is not None:  # (query token, key): head 0 of that token reads that key alone
        tok, key = point_at
        kc[int(bt[0, key // ps]), 0, key % ps] = (qkv[tok, :d].float() * 20.0).to(BF16)
    cu = torch.tensor([0, q_len], device=DEV, dtype=torch.int32)
    st = torch.tensor([start], device=DEV, dtype=torch.int32)
    got = torch.full((q_len, nh * d), float("nan"), device=DEV, dtype=BF16)
    want = torch.empty_like(got)
    scale = 1 / math.sqrt(d)
    k.paged_attention(qkv, got, kc, vc, bt, cu, st, 1, q_len, nh, nkv, d, scale, q_len, window=window, kernel=kernel)
    ref.paged_attention(qkv, want, kc, vc, bt, cu, st, 1, q_len, nh, nkv, d, scale, q_len, window=window,
                        compute_dtype=torch.float64)
    torch.cuda.synchronize()
    k.check_status()
    return got.float(), want.float(), vc, bt


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("kernel", ["tcgen05", "auto", "mma"])
def test_prompt_portion_of_8192_tokens(d, kernel):
    got, want, _, _ = _prefill_case(8192, 0, d, None, seed=d, kernel=kernel)
    torch.testing.assert_close(got, want, **TOL)


@pytest.mark.parametrize("d,window", [(128, None), (64, None), (128, 9000)])
@pytest.mark.parametrize("kernel", ["tcgen05", "auto"])
def test_prompt_portion_behind_a_30k_prefix(d, window, kernel):
    """2,048 new tokens over 30,003 cached keys (a start that is no multiple of a tile or a page):
    every query walks some 250 key tiles, the rings of the tcgen05 kernel turn over a hundred
    times, and the block table is 2,004 pages wide.  The last token's head 0 points at key 0,
    unless a window hides that key; then at the first key inside the window."""
    start, q_len = 30003, 2048
    key = 0 if window is None else start + q_len - window
    got, want, vc, bt = _prefill_case(q_len, start, d, window, seed=7 + d, kernel=kernel, point_at=(q_len - 1, key))
    torch.testing.assert_close(got, want, **TOL)
    torch.testing.assert_close(got[q_len - 1, :d], vc[int(bt[0, key // 16]), 0, key % 16].float(), **TOL)


# ---- the engine at 9 k tokens -----------------------------------------------------------------------

def _peaked_7b_layer(folder, gain=1.5):
    """One layer of the 7B geometry with a small vocabulary, random weights, and q/k projections
    scaled up so that attention is peaked: a key that went missing would move the logits.  (At
    this width random N(0, 0.02) projections already give scores of deviation 1.4; the gain
    makes it 3.2, a few dozen keys out of 9,000 then carry a row.  Much more and bfloat16
    rounding alone decides between the two best keys.)"""
    from safetensors.torch import load_file, save_file

    from emberserve_b200.config.model import Qwen2Config
    from emberserve_b200.weights.loader import write_random_model

    cfg = Qwen2Config(vocab_size=2048, hidden_size=3584, intermediate_size=18944, num_hidden_layers=1,
                      num_attention_heads=28, num_key_value_heads=4, head_dim=128, max_position_embeddings=16384,
                      rms_norm_eps=1e-6, rope_theta=1_000_000.0, tie_word_embeddings=False, attention_bias=True,
                      eos_token_ids=(1,))
    write_random_model(cfg, folder, seed=21)
    path = str(folder / "model.safetensors")
    tensors = load_file(path)
    for name in list(tensors):
        if ".q_proj." in name or ".k_proj." in name:
            tensors[name] = (tensors[name].float() * gain).to(tensors[name].dtype)
    save_file(tensors, path)
    return cfg


def _plain_logits_on_the_gpu(folder, tokens):
    """The plain implementation (tests/plain_qwen2.py) with its tensors on the GPU, in float64: at
    9 k tokens the score matrix alone is tens of GB, more than the host may have."""
    cfgd, w = plain.read_model_dir(folder)
    w = {k: v.to(DEV) for k, v in w.items()}
    out = plain.forward_logits(cfgd, w, tokens, torch.float64, device=DEV).cpu().numpy()
    del w
    torch.cuda.empty_cache()  # (tens of GB of score matrices: hand them back to the device)
    return out


def test_one_7b_layer_over_9k_tokens_under_three_cuts(tmp_path):
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner

    folder = tmp_path / "layer"
    cfg = _peaked_7b_layer(folder)
    n = 9001
    reqs = rc.make_requests(cfg.vocab_size, [n], seed=33)
    want = _plain_logits_on_the_gpu(folder, reqs[0][1])
    scale = float(np.abs(want).max())
    runner = ModelRunner.from_dir(folder, BF16, page_size=16, num_pages=-(-n // 16) + 2)
    assert runner.enable_graphs(cfg.max_position_embeddings, 4)
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 32),
            "portions of 2048": rc.portions(reqs, sizes=(2048,))}
    for cut, steps in cuts.items():
        rp = TraceReplayer(runner)
        got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
        err = np.array([np.abs(got[("r0", p)] - want[p]).max() for p in range(n)])
        worst = int(err.argmax())
        assert err[worst] <= 3e-2 * scale, f"{cut}: |dlogit| {err[worst]:.3e} at position {worst} (scale {scale:.3f})"
        runner.cache.check()
    assert 1 in runner.graphs._graphs, "the tail did not go through a CUDA graph"
