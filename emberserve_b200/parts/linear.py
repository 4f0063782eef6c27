"""Dense projections ``y = x W^T (+ b)`` of the parts.

The matrix products go to cuBLAS through ``torch.mm`` / ``torch.addmm``, where the
reference's engine uses the same library through ``nn.Linear``
(``emberserve/model/qwen2.py:57-58,77-79,203``).  Outputs land in scratch buffers of the
step, so a step allocates nothing once it is warm.

Precision: in the 32-bit path the product is a true float32 one (TF32 is switched off
for the process by ``strict_matmul_precision``); in the bfloat16 path the inputs are
bfloat16 and cuBLAS accumulates in float32, and reductions in reduced precision are
switched off.  A parameter that the checkpoint stores in 32 bits stays 32-bit: its
projection is then computed in float32 and rounded once.
"""

from __future__ import annotations

import torch


def strict_matmul_precision() -> None:
    """Process-wide matmul settings of the engine: no TF32, no split-K in bfloat16."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
           out: torch.Tensor) -> torch.Tensor:
    """out = x @ weight.T (+ bias).  x: [N, K], weight: [M, K], out: [N, M]."""
    same = weight.dtype == x.dtype and (bias is None or bias.dtype == x.dtype)
    if same and out.dtype == x.dtype:
        if bias is None:
            torch.mm(x, weight.t(), out=out)
        else:
            torch.addmm(bias, x, weight.t(), out=out)
        return out
    # A 32-bit parameter beside bfloat16 activations (or a 32-bit output): float32 product.
    y = torch.mm(x.float(), weight.float().t())
    if bias is not None:
        y += bias.float()
    out.copy_(y)
    return out


_F32_OUT_OK: bool | None = None


def linear_f32_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out (float32) = x @ weight.T with the product accumulated in float32 and never
    rounded to the activation type (the logits of the language-model head)."""
    global _F32_OUT_OK
    if x.dtype == torch.float32 and weight.dtype == torch.float32:
        torch.mm(x, weight.t(), out=out)
        return out
    if x.dtype == weight.dtype == torch.bfloat16:
        if _F32_OUT_OK is None:
            try:
                torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
                _F32_OUT_OK = True
                return out
            except (TypeError, RuntimeError):
                _F32_OUT_OK = False
        if _F32_OUT_OK:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
            return out
        out.copy_(torch.mm(x, weight.t()))
        return out
    out.copy_(torch.mm(x.float(), weight.float().t()))
    return out
