"""The tiny Qwen2 configurations of the tests.  They differ in every size and option:
head counts and groups, sizes that are no power of two, layers, vocabulary, the norms'
eps, rotary base, tied or untied head, and the window."""

from __future__ import annotations

from emberserve_b200.config.model import Qwen2Config

TINY_A = Qwen2Config(
    vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=128,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True, attention_bias=True,
    eos_token_ids=(1,))

TINY_B = Qwen2Config(
    vocab_size=320, hidden_size=96, intermediate_size=224, num_hidden_layers=3,
    num_attention_heads=3, num_key_value_heads=1, head_dim=32, max_position_embeddings=256,
    rms_norm_eps=1e-5, rope_theta=1_000_000.0, tie_word_embeddings=False, attention_bias=True,
    eos_token_ids=(2, 7))

# Sliding window in the upper layers (the lower one attends to everything), seven query
# heads on one KV head, head size 48, widths that are no power of two, no q/k/v bias.
TINY_C = Qwen2Config(
    vocab_size=203, hidden_size=112, intermediate_size=176, num_hidden_layers=3,
    num_attention_heads=7, num_key_value_heads=1, head_dim=48, max_position_embeddings=512,
    rms_norm_eps=3e-6, rope_theta=50_000.0, tie_word_embeddings=True, attention_bias=False,
    eos_token_ids=(5,), sliding_window=20, max_window_layers=1)

# Head size 64 with five query heads per KV head and a window in the top layer: the sizes
# at which the bfloat16 path runs its tensor-core attention kernels (the other three run the
# generic kernel in both paths, their head sizes being 16, 32 and 48).
TINY_D = Qwen2Config(
    vocab_size=288, hidden_size=160, intermediate_size=208, num_hidden_layers=2,
    num_attention_heads=10, num_key_value_heads=2, head_dim=64, max_position_embeddings=384,
    rms_norm_eps=1e-6, rope_theta=1_000_000.0, tie_word_embeddings=False, attention_bias=True,
    eos_token_ids=(3,), sliding_window=70, max_window_layers=1)

ALL = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D}
SEEDS = {"tiny_a": 0, "tiny_b": 1, "tiny_c": 2, "tiny_d": 3}
PAGE_SIZES = {"tiny_a": 4, "tiny_b": 8, "tiny_c": 16, "tiny_d": 16}
