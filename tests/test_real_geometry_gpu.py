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
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


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
    runner = ModelRunner.from_dir(folder, dtype, page_size=16, num_pages=40)
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
