"""Qwen2 / Qwen2.5 dense (``Qwen2ForCausalLM``) as an assembly of parts.

Every layer is a pre-norm block of grouped-query attention (q/k/v bias, rotate-half
rotary encoding over the full head) and a SwiGLU feed-forward, between RMSNorms; one
shared rotary table; final RMSNorm; a head that is the embedding when
``tie_word_embeddings`` (``emberserve/model/qwen2.py:64-230``).  Checkpoint names are
Hugging Face's (``emberserve/model/weights.py:25-33`` fuses q/k/v and gate/up the same
way).  Layers at or past ``max_window_layers`` get the sliding window when the config
switches it on, so the layers of one model may have different cache needs.
"""

from __future__ import annotations

from emberserve_b200.config.model import Qwen2Config
from emberserve_b200.parts.attention import AttentionSpec
from emberserve_b200.parts.block import PreNormBlockSpec
from emberserve_b200.parts.decoder import DecoderSpec, LayerCall
from emberserve_b200.parts.mlp import SwiGLUSpec
from emberserve_b200.parts.norm import RMSNormSpec
from emberserve_b200.parts.rope import RotarySpec
from emberserve_b200.registry import register_architecture


def build_qwen2_spec(cfg: Qwen2Config) -> DecoderSpec:
    rotary = RotarySpec(rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                        max_positions=cfg.max_position_embeddings)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(PreNormBlockSpec(
            mixer=AttentionSpec(
                hidden=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                qkv_bias=cfg.attention_bias, position=rotary,
                q_name=f"{p}.self_attn.q_proj", k_name=f"{p}.self_attn.k_proj",
                v_name=f"{p}.self_attn.v_proj", o_name=f"{p}.self_attn.o_proj",
                window=cfg.layer_window(i)),
            feed_forward=SwiGLUSpec(
                hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                gate_name=f"{p}.mlp.gate_proj", up_name=f"{p}.mlp.up_proj",
                down_name=f"{p}.mlp.down_proj"),
            mixer_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, f"{p}.input_layernorm.weight"),
            ffn_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps,
                                 f"{p}.post_attention_layernorm.weight"),
        ))
    ignorable = ("rotary_emb.inv_freq",)
    if cfg.tie_word_embeddings:
        ignorable += ("lm_head.weight",)  # a tied checkpoint may still carry the copy
    return DecoderSpec(
        vocab_size=cfg.vocab_size, hidden=cfg.hidden_size,
        embed_name="model.embed_tokens.weight",
        layers=layers,
        order=[LayerCall(layer=i, cache=i) for i in range(cfg.num_hidden_layers)],
        final_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_positions=cfg.max_position_embeddings,
        ignorable=ignorable,
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, build_qwen2_spec, model_types=("qwen2",))
