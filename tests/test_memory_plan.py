"""The division of device memory between the cache and the steps (engine/memory.py), against
numbers worked out by hand for the real shapes, and the options the engine derives from its
configuration."""

from __future__ import annotations

import dataclasses

import pytest
import torch

from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.config.model import Qwen2Config
from emberserve_b200.engine.llm_engine import LLMEngine
from emberserve_b200.engine.memory import WORKSPACE_BYTES, plan_memory
from emberserve_b200.registry import build_decoder

GIB = 1 << 30


def _shape(hidden, inter, layers, heads, kv_heads, vocab, tied, head_dim=None):
    return Qwen2Config.from_dict({
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab, "hidden_size": hidden,
        "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "tie_word_embeddings": tied, **({"head_dim": head_dim} if head_dim else {})})


SHAPES = {
    # name: (config, hand-computed bytes of step scratch per token in bfloat16, bytes of one 16-token page)
    # per token: 4 H (float32 residual) + 2 * [attention (q + 2 kv) + q + H; feed-forward 3 I + H; norm H]
    "0.5b": (_shape(896, 4864, 24, 14, 2, 151936, True),
             4 * 896 + 2 * ((896 + 256 + 896 + 896) + (3 * 4864 + 896) + 896),
             24 * 2 * 2 * 16 * 64 * 2),
    "7b": (_shape(3584, 18944, 28, 28, 4, 152064, False),
           165888,  # = 14336 + 2 * (11776 + 60416 + 3584)
           28 * 2 * 4 * 16 * 128 * 2),
    "32b": (_shape(5120, 27648, 64, 40, 8, 152064, False),
            4 * 5120 + 2 * ((5120 + 2048 + 5120 + 5120) + (3 * 27648 + 5120) + 5120),
            64 * 2 * 8 * 16 * 128 * 2),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_scratch_per_token_of_the_real_shapes(name):
    cfg, per_token, _ = SHAPES[name]
    assert build_decoder(cfg).scratch_bytes_per_token(2) == per_token


def test_plan_for_the_7b_shape_by_hand():
    cfg, per_token, page = SHAPES["7b"]
    assert page == 917504
    free = 160 * GIB
    plan = plan_memory(free_bytes=free, utilization=0.9, bytes_per_page=page, scratch_bytes_per_token=per_token,
                       vocab_size=cfg.vocab_size, max_step_tokens=8192, max_logit_rows=256, graph_rows=256)
    assert plan.workspace == WORKSPACE_BYTES == 1073741824
    assert plan.step_scratch == 8192 * 165888 == 1358954496
    assert plan.step_logits == plan.graph_logits == 256 * 152064 * 4 == 155713536
    assert plan.graph_scratch == 256 * 165888 == 42467328
    assert plan.reserve == 2786590720
    assert plan.num_pages == (int(free * 0.9) - 2786590720) // 917504 == 165484
    assert plan.cache_bytes <= int(free * 0.9) - plan.reserve < plan.cache_bytes + page


@pytest.mark.parametrize("name,util,free_gib,step_tokens,rows", [
    ("0.5b", 0.90, 170, 8192, 256), ("32b", 0.97, 110, 2048, 32), ("7b", 0.97, 165, 8192, 256)])
def test_plan_terms_of_the_other_shapes(name, util, free_gib, step_tokens, rows):
    cfg, per_token, page = SHAPES[name]
    free = free_gib * GIB
    plan = plan_memory(free_bytes=free, utilization=util, bytes_per_page=page, scratch_bytes_per_token=per_token,
                       vocab_size=cfg.vocab_size, max_step_tokens=step_tokens, max_logit_rows=rows, graph_rows=rows)
    hand = GIB + step_tokens * per_token + 2 * rows * cfg.vocab_size * 4 + rows * per_token
    assert plan.reserve == hand
    assert plan.num_pages == (int(free * util) - hand) // page
    # what is left after the cache and the reserve is less than a page plus the share kept unused
    assert free - plan.cache_bytes - plan.reserve < free * (1 - util) + page + 1


def test_no_graphs_no_graph_terms_and_an_override():
    cfg, per_token, page = SHAPES["0.5b"]
    plan = plan_memory(free_bytes=8 * GIB, utilization=0.9, bytes_per_page=page, scratch_bytes_per_token=per_token,
                       vocab_size=cfg.vocab_size, max_step_tokens=1024, max_logit_rows=16, graph_rows=0,
                       state_bytes=12345)
    assert plan.graph_scratch == plan.graph_logits == 0 and plan.state == 12345
    assert plan.reserve == GIB + 1024 * per_token + 16 * cfg.vocab_size * 4 + 12345
    fixed = plan_memory(free_bytes=8 * GIB, utilization=0.9, bytes_per_page=page, scratch_bytes_per_token=per_token,
                        vocab_size=cfg.vocab_size, max_step_tokens=1024, max_logit_rows=16, graph_rows=0,
                        reserve_override=2 * GIB)
    assert fixed.num_pages == (int(8 * GIB * 0.9) - 2 * GIB) // page
    # less memory than the reserve: no pages (the runner then falls back to its floor)
    assert plan_memory(free_bytes=GIB, utilization=0.9, bytes_per_page=page, scratch_bytes_per_token=per_token,
                       vocab_size=cfg.vocab_size, max_step_tokens=8192, max_logit_rows=256,
                       graph_rows=256).num_pages == 0


def test_runner_options_follow_the_engine_configuration():
    cfg = EngineConfig(max_num_seqs=48, max_num_batched_tokens=512, max_model_len=2000, block_size=16,
                       gpu_memory_utilization=0.8)
    opt = LLMEngine.runner_options(cfg)
    assert opt["max_step_tokens"] == 512 and opt["max_graph_rows"] == 48 and opt["max_logit_rows"] == 48
    assert opt["max_pages"] == 48 * 125 and opt["num_state_slots"] == 48 and opt["gpu_memory_utilization"] == 0.8
    # without chunked prefill a preempted request returns whole: up to max_model_len tokens in a step
    whole = LLMEngine.runner_options(dataclasses.replace(cfg, enable_chunked_prefill=False))
    assert whole["max_step_tokens"] == 2000
    assert LLMEngine.runner_options(dataclasses.replace(cfg, enable_cuda_graphs=False))["max_graph_rows"] == 0
    assert cfg.max_num_batched_tokens == 512  # (the configuration itself is never changed)
