"""Pre-norm residual block: ``h += mixer(norm1(h)); h += ffn(norm2(h))``.

Written on the pair (delta, residual) so that each norm performs the add that precedes
it (``emberserve/model/qwen2.py:122-164``): the block receives the previous block's
output `delta`, which has not been added to the stream yet, and returns its own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200.parts.base import (Block, CacheNeed, Part, StepContext, build_part,
                                        register_part)


@dataclass(frozen=True)
class PreNormBlockSpec:
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    ffn_norm: Any
    kind: str = "prenorm"


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: PreNormBlockSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        self.mixer_norm = build_part("norm", spec.mixer_norm, prefix + ".mixer_norm", self.shared)
        self.mixer = build_part("mixer", spec.mixer, prefix + ".mixer", self.shared)
        self.ffn_norm = build_part("norm", spec.ffn_norm, prefix + ".ffn_norm", self.shared)
        self.ffn = build_part("feed_forward", spec.feed_forward, prefix + ".ffn", self.shared)

    def children(self) -> dict[str, Part]:
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def cache_need(self) -> CacheNeed | None:
        return self.mixer.cache_need()

    def entry_norm(self):
        return self.mixer_norm if self.mixer.splits_norms else None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                cache: Any) -> torch.Tensor:
        # A sub-layer whose successor takes `ScaledRows` is asked to begin the norm that follows
        # it in its last product (ctx.extra["norm_behind"]); what it returns says whether it did.
        after_ffn = ctx.extra.pop("next_norm", None)  # the next block's entry norm, from the decoder
        x = self.mixer_norm.forward(delta, residual, ctx)
        ctx.extra["norm_behind"] = (self.ffn_norm.split_request(residual, ctx)
                                    if self.mixer.splits_norms and self.ffn.splits_norms else None)
        a = self.mixer.forward(x, ctx, cache)
        y = self.ffn_norm.forward(a, residual, ctx)
        ctx.extra["norm_behind"] = (after_ffn.split_request(residual, ctx)
                                    if after_ffn is not None and self.ffn.splits_norms else None)
        out = self.ffn.forward(y, ctx)
        ctx.extra["norm_behind"] = None
        return out
