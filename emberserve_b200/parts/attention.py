"""Grouped-query causal attention over a paged cache (the mixer of Qwen2).

``qkv = x Wqkv^T + b`` with columns ``[q | k | v]`` (``emberserve/model/qwen2.py:70-78,
93-100``), rotary encoding of q and k, write of k and v into the cache pages, causal
softmax attention of every query over its request's keys with query head h reading KV
head ``h // groups`` and scale ``1/sqrt(head_dim)`` (``emberserve/attn/base.py:105-128``),
then ``o = attn Wo^T`` without bias (``qwen2.py:113-114``).  A window of W keys, if the
spec has one, hides keys at positions ``<= p - W`` from the query at position p.

The part never touches the cache manager: it gets a ``PagedKVHandle`` for the step and
hands the block tables to the kernels (``attn/base.py:79-91`` is the same contract).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Mixer, PagedKV, PagedKVHandle, ParamSpec, Source,
                                        StepContext, register_part)
from emberserve_b200.parts.linear import linear

# Blocks wanted in flight before keys are split among several blocks of a decode step:
# this many per SM of the device.
_BLOCKS_PER_SM = 2
_MAX_SPLITS = 64
_MIN_KEYS_PER_SPLIT = 128


_log = logging.getLogger("emberserve_b200")
_slow_path_told: set[tuple[int, int]] = set()


def _tell_slow_path_once(head_dim: int, group: int) -> None:
    """One line, once per geometry, when bfloat16 attention cannot run on the tensor-core
    kernels (head sizes 64 and 128; at most 16 query heads per KV head in decode steps) and
    takes the 32-bit CUDA-core kernel instead: right, but several times slower."""
    key = (head_dim, group)
    if key not in _slow_path_told:
        _slow_path_told.add(key)
        _log.warning("bfloat16 attention with head_dim=%d and %d query heads per KV head runs on the generic "
                     "CUDA-core kernel: the tensor-core kernels take head sizes 64 and 128 (and up to 16 heads "
                     "per KV head when decoding)", head_dim, group)


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: Any  # spec of a position encoding (rotary), or None
    # checkpoint names of the four projections, without ".weight" / ".bias"
    q_name: str
    k_name: str
    v_name: str
    o_name: str
    window: int | None = None
    scale: float | None = None  # None = head_dim ** -0.5
    kind: str = "gqa_attention"


def decode_splits(num_rows: int, num_kv_heads: int, max_ctx: int, sms: int | None = None) -> int:
    """How many blocks share the keys of one (request, KV head) in a decode step.  A
    function of shapes and of the device's SM count `sms` only
    (``emberserve/attn/paged_triton.py:259-281`` has the same idea)."""
    blocks = max(1, num_rows * num_kv_heads)
    target = _BLOCKS_PER_SM * (sms if sms is not None else K.sm_count())
    want = target // blocks  # rounded down: all blocks of the step run in one wave
    cap = max(1, max_ctx // _MIN_KEYS_PER_SPLIT)
    return max(1, min(_MAX_SPLITS, want, cap))


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    splits_norms = True
    wqkv: torch.Tensor
    wo: torch.Tensor
    bqkv: torch.Tensor | None = None

    def __init__(self, spec: AttentionSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"head_dim={spec.head_dim}: the attention kernels take multiples "
                             f"of 16 up to 256")
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5
        self.position = self.shared.get("position", spec.position) if spec.position is not None else None

    def cache_need(self) -> PagedKV:
        s: AttentionSpec = self.spec
        return PagedKV(s.num_kv_heads, s.head_dim, s.window)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: AttentionSpec = self.spec
        q, kv = self.q_size, self.kv_size
        rows = [(s.q_name, (0, q)), (s.k_name, (q, q + kv)), (s.v_name, (q + kv, q + 2 * kv))]
        specs = {
            "wqkv": ParamSpec((q + 2 * kv, s.hidden), [Source(n + ".weight", r) for n, r in rows]),
            "wo": ParamSpec((s.hidden, q), [Source(s.o_name + ".weight")]),
        }
        if s.qkv_bias:
            specs["bqkv"] = ParamSpec((q + 2 * kv,), [Source(n + ".bias", r) for n, r in rows],
                                      init="bias")
        return specs

    def streamed_params(self) -> list[str]:
        return ["wqkv", "wo"]

    def scratch_elements_per_token(self) -> int:
        # qkv, attn_out, mixer_out
        return self.q_size + 2 * self.kv_size + self.q_size + self.spec.hidden

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVHandle) -> torch.Tensor:
        s: AttentionSpec = self.spec
        n = ctx.num_tokens
        qkv = ctx.scratch("qkv", (n, self.q_size + 2 * self.kv_size), ctx.dtype)
        linear(x, self.wqkv, self.bqkv, qkv, ctx.scratch)
        behind = ctx.extra.get("norm_behind")  # the norm behind this mixer, if wo's product may begin it
        table, rot = (None, 0)
        if self.position is not None:
            r = self.position.rotary(ctx.device)
            if r is not None:
                table, rot = r
        b = ctx.num_rows
        kern = ctx.extra.get("attn_kernel", "auto")  # the engine's choice of attention kernels
        if (ctx.dtype == torch.bfloat16 and kern != "generic"
                and (s.head_dim not in (64, 128) or s.num_heads // s.num_kv_heads > 16)):
            _tell_slow_path_once(s.head_dim, s.num_heads // s.num_kv_heads)
        if (kern != "generic" and ctx.all_decode and n == b and x.is_cuda
                and K.decode_attention_fused_supported(ctx.dtype, s.num_heads, s.num_kv_heads, s.head_dim, rot)):
            # a decode step in bfloat16: rotation, cache write and attention in one kernel
            out = ctx.scratch("attn_out", (n, self.q_size), ctx.dtype)
            # (in a captured step ctx.max_ctx_len is the longest context its graph serves, so
            # the split is fixed per bucket and per layer)
            splits = decode_splits(b, s.num_kv_heads, ctx.max_ctx_len, K.sm_count(ctx.device))
            scratch = None
            if splits > 1:
                nbytes = K.attention_scratch_bytes(b, s.num_heads, s.head_dim, splits)
                scratch = ctx.scratch("attn_partials", (nbytes // 4,), torch.float32)
            K.decode_attention_fused(qkv, out, cache.k, cache.v, cache.block_tables, ctx.cu_q, ctx.starts, b,
                                     s.num_heads, s.num_kv_heads, s.head_dim, self.scale, table, rot,
                                     cache.write, window=cache.window, splits=splits, scratch=scratch)
            y = ctx.scratch("mixer_out", (n, s.hidden), ctx.dtype)
            return linear(out, self.wo, None, y, ctx.scratch, behind)
        K.rope_kv_write(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx.positions,
                        ctx.row_of_token, table, rot, cache.k, cache.v, cache.block_tables,
                        cache.page_size, write_kv=cache.write)
        out = ctx.scratch("attn_out", (n, self.q_size), ctx.dtype)
        # Rows that bring one token and stand first (the scheduler puts decoding requests
        # first) go to the split-key decode kernel; the rest, prompt portions, follow.
        nd = 0
        while nd < b and ctx.q_lens[nd] == 1:
            nd += 1
        if nd > 0:
            splits, scratch = 1, None
            max_ctx = ctx.max_ctx_len if nd == b else max(st + 1 for st in ctx.start_list[:nd])
            splits = decode_splits(nd, s.num_kv_heads, max_ctx, K.sm_count(ctx.device))
            if splits > 1:
                nbytes = K.attention_scratch_bytes(nd, s.num_heads, s.head_dim, splits)
                scratch = ctx.scratch("attn_partials", (nbytes // 4,), torch.float32)
            K.paged_attention(qkv, out, cache.k, cache.v, cache.block_tables[:nd], ctx.cu_q[:nd + 1],
                              ctx.starts[:nd], nd, nd, s.num_heads, s.num_kv_heads, s.head_dim,
                              self.scale, 1, window=cache.window, splits=splits, scratch=scratch, kernel=kern)
        if nd < b:
            K.paged_attention(qkv, out, cache.k, cache.v, cache.block_tables[nd:], ctx.cu_q[nd:],
                              ctx.starts[nd:], b - nd, n, s.num_heads, s.num_kv_heads, s.head_dim,
                              self.scale, max(ctx.q_lens[nd:]), window=cache.window, kernel=kern)
        y = ctx.scratch("mixer_out", (n, s.hidden), ctx.dtype)
        return linear(out, self.wo, None, y, ctx.scratch, behind)
