"""The layer sizes of real Qwen2.5 checkpoints (0.5B, 7B, 32B: widths, head counts, groups,
head sizes, feed-forward widths) with few layers and a small vocabulary, random weights, in
32-bit and in bfloat16, under the four ways of cutting, against the plain implementation.
At these sizes the bfloat16 path runs its tensor-core attention kernels and, for rows that
bring one token, the tcgen05 projection kernels; the tiny configurations mostly do not."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_cases as rc

from emberserve_b200.config.model import Qwen2Config

pytestmark = pytest.mark.gpu

SHAPES = {
    # name: (hidden, heads, kv_heads, head_dim, intermediate, layers, eps, tied)
    "qwen2.5-0.5b": (896, 14, 2, 64, 4864, 2, 1e-6, True),
    "qwen2.5-7b": (3584, 28, 4, 128, 18944, 1, 1e-6, False),
    "qwen2.5-32b": (5120, 40, 8, 128, 27648, 1, 1e-5, False),
}
LENGTHS = [70, 150, 40, 97]
TOL = {torch.float32: 3e-5, torch.bfloat16: 1.5e-2}


def config_of(name: str) -> Qwen2Config:
    h, nh, nkv, d, inter, layers, eps, tied = SHAPES[name]
    return Qwen2Config(vocab_size=2048, hidden_size=h, intermediate_size=inter, num_hidden_layers=layers,
                       num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d,
                       max_position_embeddings=1024, rms_norm_eps=eps, rope_theta=1_000_000.0,
                       tie_word_embeddings=tied, attention_bias=True, eos_token_ids=(1,))


@pytest.fixture(scope="module", params=list(SHAPES))
def case(request, tmp_path_factory):
    from emberserve_b200.weights.loader import write_random_model

    name = request.param
    cfg = config_of(name)
    folder = write_random_model(cfg, tmp_path_factory.mktemp(name.replace(".", "_")), seed=11)
    reqs = rc.make_requests(cfg.vocab_size, LENGTHS, seed=3)
    cfgd, w = plain.read_model_dir(folder)
    oracle_dtype = torch.float64 if name != "qwen2.5-32b" else torch.float32  # memory of the host
    want = {rid: plain.forward_logits(cfgd, w, toks, oracle_dtype).double().numpy() for rid, toks in reqs}
    return name, folder, reqs, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_real_layer_sizes_under_every_cut(case, dtype):
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner
    from emberserve_b200 import kernels as K

    name, folder, reqs, want = case
    scale = max(float(np.abs(v).max()) for v in want.values())
    # (guard elements around every scratch buffer: a kernel that writes outside its buffer at
    # these sizes is caught by verify_scratch below)
    runner = ModelRunner.from_dir(folder, dtype, page_size=16, num_pages=40, scratch_guard=64)
    runner.enable_graphs(1024, 4)
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 32), "portions": rc.portions(reqs),
            "mixed": rc.mixed(reqs, max_live=3, seed=5, decode_tail=16)}
    for cut, steps in cuts.items():
        assert rc.max_live_tokens(steps) <= 40 * 16
        rp = TraceReplayer(runner)
        got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
        torch.cuda.synchronize()
        K.check_status()
        worst = max(float(np.abs(got[(rid, p)] - want[rid][p]).max())
                    for rid, toks in reqs for p in range(len(toks)))
        assert worst <= TOL[dtype] * scale, f"{name} {cut} {dtype}: {worst:.3e} vs scale {scale:.3f}"
        runner.cache.check()
        runner.verify_scratch()


@pytest.mark.parametrize("name", ["qwen2.5-0.5b", "qwen2.5-7b"])
def test_long_prompt_through_the_tcgen05_attention(name, tmp_path):
    """A prompt long enough that its portions go to the tcgen05 attention kernel (at least 2048
    query rows per KV head): whole in one step, and in portions that start behind a cached prefix
    at positions that are no multiple of the key tile, beside a short request; bfloat16 against
    the plain implementation in float32."""
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner
    from emberserve_b200.weights.loader import write_random_model
    from emberserve_b200 import kernels as K

    cfg = config_of(name)
    folder = write_random_model(cfg, tmp_path / "m", seed=12)
    g = torch.Generator().manual_seed(5)
    long_toks = torch.randint(0, cfg.vocab_size, (700,), generator=g).tolist()
    short_toks = torch.randint(0, cfg.vocab_size, (9,), generator=g).tolist()
    cfgd, w = plain.read_model_dir(folder)
    want_long = plain.forward_logits(cfgd, w, long_toks, torch.float32).double().numpy()
    want_short = plain.forward_logits(cfgd, w, short_toks, torch.float32).double().numpy()
    scale = float(np.abs(want_long).max())
    probe = [0, 127, 128, 399, 400, 401, 402, 699]
    runner = ModelRunner.from_dir(folder, torch.bfloat16, page_size=16, num_pages=64, scratch_guard=64)
    cuts = {
        "whole": [[("L", 0, 700, probe)]],
        "portions": [[("L", 0, 400, [p for p in probe if p < 400])],
                     [("S", 0, 9, [8]), ("L", 400, 402, [0, 1])],
                     [("L", 402, 700, [0, 297])]],
    }
    for cut, plan in cuts.items():
        rp = TraceReplayer(runner)
        for i, step in enumerate(plan):
            entries = []
            for rid, a, b, want in step:
                toks = long_toks if rid == "L" else short_toks
                entries.append({"id": rid, "tokens": toks[a:b], "want": want})
            last = i == len(plan) - 1
            got = rp.run_step({"step": i, "entries": entries, "end": ["L", "S"] if last and cut == "portions" else (["L"] if last else [])})
            row = 0
            for rid, a, b, want in step:
                ref = want_long if rid == "L" else want_short
                for wpos in want:
                    err = float(np.abs(got[row] - ref[a + wpos]).max())
                    assert err <= TOL[torch.bfloat16] * scale, f"{name} {cut} step {i} {rid}@{a + wpos}: {err:.3e}"
                    row += 1
        torch.cuda.synchronize()
        K.check_status()
        runner.cache.check()
        runner.verify_scratch()


@pytest.mark.parametrize("name", ["qwen2.5-0.5b", "qwen2.5-7b"])
def test_tiled_weight_copies_change_no_logit(name, tmp_path):
    """The engine's second, tiled copy of the projection weights (made by default where it is
    small beside the device's memory) feeds the decode kernels the same numbers: the logits of
    prompt portions and of decode steps of 1, 8 and 40 rows are the same bits with and without it."""
    from emberserve_b200.engine.runner import ModelRunner, StepRow
    from emberserve_b200.weights.loader import write_random_model
    from emberserve_b200 import kernels as K

    cfg = config_of(name)
    folder = write_random_model(cfg, tmp_path / "m", seed=21)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist()
               for n in torch.randint(3, 60, (40,), generator=g)]
    got = {}
    for copies in (False, None, True):
        runner = ModelRunner.from_dir(folder, torch.bfloat16, page_size=16, num_pages=40 * 5 + 8,
                                      tiled_weight_copies=copies)
        if copies is False:
            assert runner.tiled_weight_bytes == 0
        else:  # (None: a model this small is far below a tenth of the memory)
            twins = sum(w.numel() * 2 for w in runner.decoder.streamed_weights())
            assert runner.tiled_weight_bytes == twins > 0
        outs = []
        for i, p in enumerate(prompts):
            runner.cache.admit(i, len(p) + 8)
        outs.append(runner.step([StepRow(i, p, 0, [len(p) - 1]) for i, p in enumerate(prompts)]).clone())
        for rows in (1, 8, 40):
            for step in range(2):
                batch = [StepRow(i, [7 + i + step], runner.cache.committed(i), [0]) for i in range(rows)]
                outs.append(runner.step(batch).clone())
        torch.cuda.synchronize()
        K.check_status()
        got[copies] = outs
    for a, b, c in zip(got[False], got[None], got[True]):
        assert torch.equal(a, b) and torch.equal(a, c)
