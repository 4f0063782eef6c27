"""Dense gated feed-forward (SwiGLU): ``down(silu(gate(x)) * up(x))``, no biases.

gate and up are one fused projection whose first I output columns are the gate and the
last I the up part (``emberserve/model/qwen2.py:48-61``); the activation is
``silu(g) * u`` computed in 32 bits (``emberserve/model/ops.py:84-87``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import FeedForward, ParamSpec, Source, StepContext, register_part
from emberserve_b200.parts.linear import gated_linear, linear


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    # checkpoint names of the three projections, without ".weight"
    gate_name: str
    up_name: str
    down_name: str
    kind: str = "swiglu"


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    splits_norms = True
    wgu: torch.Tensor
    wdown: torch.Tensor

    def param_specs(self) -> dict[str, ParamSpec]:
        s: SwiGLUSpec = self.spec
        i = s.intermediate
        return {
            "wgu": ParamSpec((2 * i, s.hidden), [Source(s.gate_name + ".weight", (0, i)),
                                                 Source(s.up_name + ".weight", (i, 2 * i))]),
            "wdown": ParamSpec((s.hidden, i), [Source(s.down_name + ".weight")]),
        }

    def streamed_params(self) -> list[str]:
        return ["wgu", "wdown"]

    def scratch_elements_per_token(self) -> int:
        # ffn_act, ffn_out, and gate_up for the steps in which no fused kernel takes the sizes
        return 3 * self.spec.intermediate + self.spec.hidden

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        s: SwiGLUSpec = self.spec
        n = x.shape[0]
        act = ctx.scratch("ffn_act", (n, s.intermediate), ctx.dtype)
        if not gated_linear(x, self.wgu, act):  # both projections and SiLU in one kernel, where one takes the sizes
            gu = ctx.scratch("gate_up", (n, 2 * s.intermediate), ctx.dtype)
            linear(x, self.wgu, None, gu, ctx.scratch)
            K.silu_mul(gu, act)
        y = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
        # (the norm behind this feed-forward, if the down projection's product may begin it)
        return linear(act, self.wdown, None, y, ctx.scratch, ctx.extra.get("norm_behind"))
