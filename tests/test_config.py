"""Typed configuration and the architecture registry."""

from __future__ import annotations

import json

import pytest

from tiny_configs import ALL, TINY_B

from emberserve_b200.config.engine import EngineConfig, dtype_from_str
from emberserve_b200.config.model import ConfigError, Qwen2Config
from emberserve_b200.registry import (build_decoder, load_config, registered_architectures,
                                      resolve_architecture)

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 152064,
    "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "max_position_embeddings": 32768,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False,
    "sliding_window": 131072, "use_sliding_window": False, "max_window_layers": 28,
    "eos_token_id": 151645, "bos_token_id": 151643, "hidden_act": "silu", "torch_dtype": "bfloat16"}


def test_real_shape_parses_with_defaults():
    cfg = Qwen2Config.from_dict(QWEN25_7B)
    assert cfg.head_dim == 128 and cfg.num_kv_groups == 7 and cfg.attention_bias
    assert cfg.sliding_window is None  # present in the file but switched off: accepted
    assert cfg.eos_token_ids == (151645,) and cfg.bos_token_id == 151643
    assert cfg.kv_bytes_per_token(2) == 57344
    assert abs(cfg.num_parameters() - 7.6e9) < 0.1e9


def test_defaults_of_optional_keys():
    cfg = Qwen2Config.from_dict({"vocab_size": 10, "hidden_size": 32, "intermediate_size": 8,
                                 "num_hidden_layers": 1, "num_attention_heads": 2})
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps, cfg.rope_theta) == (2, 16, 1e-6, 1e6)
    assert cfg.tie_word_embeddings and cfg.attention_bias and cfg.eos_token_ids == (151645,)
    assert cfg.max_position_embeddings == 32768


@pytest.mark.parametrize("name", list(ALL))
def test_round_trip_through_config_json(tmp_path, name):
    cfg = ALL[name]
    cfg.save(tmp_path)
    assert load_config(tmp_path) == cfg
    assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]


@pytest.mark.parametrize("change,match", [
    ({"model_type": "llama", "architectures": ["LlamaForCausalLM"]}, "unsupported architecture"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"num_key_value_heads": 2}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"vocab_size": None}, "vocab_size"),
    ({"hidden_size": 0}, "positive"),
])
def test_refusals(change, match):
    cfg = dict(TINY_B.to_dict(), **change)
    with pytest.raises(ConfigError, match=match):
        resolve_architecture(cfg).config_cls.from_dict(cfg)


def test_window_keys():
    d = dict(TINY_B.to_dict(), sliding_window=8, use_sliding_window=True, max_window_layers=2)
    cfg = Qwen2Config.from_dict(d)
    assert [cfg.layer_window(i) for i in range(3)] == [None, None, 8]
    needs = build_decoder(cfg).cache_entries()
    assert [n.window for n in needs] == [None, None, 8]
    assert Qwen2Config.from_dict(dict(d, use_sliding_window=False)).sliding_window is None


def test_registry_and_model_type_fallback():
    assert "Qwen2ForCausalLM" in registered_architectures()
    d = TINY_B.to_dict()
    d.pop("architectures")
    assert resolve_architecture(d).name == "Qwen2ForCausalLM"


def test_decoder_is_built_from_config_sizes():
    cfg = TINY_B
    table = build_decoder(cfg).param_table()
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    assert table["layers.2.mixer.wqkv"].shape == (q + 2 * kv, cfg.hidden_size)
    assert table["layers.0.ffn.wgu"].shape == (2 * cfg.intermediate_size, cfg.hidden_size)
    assert table["head"].shape == (cfg.vocab_size, cfg.hidden_size)
    assert "head" not in build_decoder(ALL["tiny_a"]).param_table()  # tied


def test_engine_config():
    assert dtype_from_str("bf16") == dtype_from_str("bfloat16")
    with pytest.raises(ValueError):
        dtype_from_str("float16")
    with pytest.raises(ValueError):
        EngineConfig(block_size=0)
    assert EngineConfig(dtype="float32").dtype == dtype_from_str("fp32")
    assert EngineConfig().attn_backend == "auto" and EngineConfig(attn_backend="generic").attn_backend == "generic"
    with pytest.raises(ValueError, match="attn_backend"):
        EngineConfig(attn_backend="paged_flash")
    assert EngineConfig().debug_scratch_guard == 0


def test_command_line_options_map_to_the_engine_configuration():
    """The reference's option names (emberserve/cli.py:12-66) with this engine's choices."""
    from emberserve_b200.cli import build_parser, engine_config_from_args

    args = build_parser().parse_args(["generate", "--model", "m", "--prompt-ids", "1,2", "--dtype", "float32",
                                      "--block-size", "32", "--num-blocks", "77", "--max-num-seqs", "9",
                                      "--max-model-len", "512", "--attn-backend", "mma", "--no-cuda-graphs",
                                      "--no-async-scheduling", "--debug-scratch-guard", "16", "--no-chunked-prefill"])
    cfg = engine_config_from_args(args)
    assert (cfg.block_size, cfg.num_gpu_blocks, cfg.max_num_seqs, cfg.max_model_len) == (32, 77, 9, 512)
    assert cfg.attn_backend == "mma" and not cfg.enable_cuda_graphs and not cfg.async_scheduling
    assert cfg.debug_scratch_guard == 16 and not cfg.enable_chunked_prefill
    assert cfg.max_num_batched_tokens == 8192  # 2048 with chunked prefill, as in the reference
    chunked = engine_config_from_args(build_parser().parse_args(["generate", "--model", "m", "--prompt", "x", "--chat"]))
    assert chunked.enable_chunked_prefill and chunked.max_num_batched_tokens == 2048 and chunked.attn_backend == "auto"
    assert chunked.enable_cuda_graphs and chunked.async_scheduling  # on unless switched off
    # the reference's switches that turn on what is on here by default are accepted as they are
    same = engine_config_from_args(build_parser().parse_args(
        ["generate", "--model", "m", "--prompt", "x", "--enable-cuda-graphs", "--async-scheduling",
         "--enable-chunked-prefill"]))
    assert same.enable_cuda_graphs and same.async_scheduling and same.enable_chunked_prefill
