"""RMSNorm fused with the residual add that precedes it.

``y = weight * cast(r * rsqrt(mean(r^2) + eps))`` with ``r = residual + delta``
(``emberserve/model/ops.py:51-63``, ``emberserve/model/qwen2.py:30-45``).  The residual
stream is held in 32 bits; the sum and the statistics are 32-bit.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Norm, NormRequest, ParamSpec, ScaledRows, Source, StepContext,
                                        register_part)


# EMBERSERVE_SPLIT_NORMS=0 keeps the norm a kernel of its own in every step (for comparisons).
_SPLIT_NORMS = os.environ.get("EMBERSERVE_SPLIT_NORMS", "1") != "0"


@dataclass(frozen=True)
class RMSNormSpec:
    dim: int
    eps: float
    weight_name: str  # checkpoint tensor of the gain, [dim]
    kind: str = "rmsnorm"


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    weight: torch.Tensor

    def param_specs(self) -> dict[str, ParamSpec]:
        s: RMSNormSpec = self.spec
        return {"weight": ParamSpec((s.dim,), [Source(s.weight_name)], init="ones")}

    def scratch_elements_per_token(self) -> int:
        return self.spec.dim  # "normed" (the rows before the head are fewer)

    def split_request(self, residual: torch.Tensor, ctx: StepContext) -> NormRequest | None:
        # In bfloat16 steps of few rows the norm is split between the products around it: the one
        # before adds into the residual, applies the gain and begins the sum of squares, the one
        # behind multiplies its rows by rsqrt(mean + eps).  (Roundings then differ from the
        # kernel's: residual * gain is rounded once, the scale is applied to a float32 result.)
        if (ctx.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and residual.is_cuda
                and ctx.num_tokens <= K.GEMM_NORM_ROWS and _SPLIT_NORMS):
            return NormRequest(residual, self.weight, self.spec.eps)
        return None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        if isinstance(delta, ScaledRows):  # begun by the product before: the product behind finishes it
            assert rows is None
            return delta
        s: RMSNormSpec = self.spec
        n = residual.shape[0] if rows is None else rows.numel()
        out = ctx.scratch("normed" if rows is None else "normed_rows", (n, s.dim), ctx.dtype)
        K.add_rmsnorm(delta, residual, self.weight, out, s.eps, rows=rows)
        return out
