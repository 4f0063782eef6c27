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

from emberserve_b200 import kernels as K


def strict_matmul_precision() -> None:
    """Process-wide matmul settings of the engine: no TF32, no split-K in bfloat16."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


_MIN_K_TILES_PER_SPLIT = 8
# Up to this many rows the hand-written kernel is used; with more, cuBLAS is as fast or faster
# (measured at the projection shapes of a 7B model).
_SMALLM_ROWS = 16
# The gate/up product with SiLU in its epilogue stays ahead up to the kernel's 64 rows: cuBLAS
# needs a separate activation kernel behind it (decode step of the 7B shape at 24 / 32 / 64 rows:
# 4.05 / 4.37 / 5.51 ms against 4.25 / 4.48 / 5.65).
_GATED_ROWS = 64


def smallm_ksplit(m_tok: int, n_out: int, k: int, sms: int | None = None) -> int:
    """Over how many blocks (one thread-block cluster, at most 8) the small-row kernel splits
    K so that the blocks of the product fill the `sms` SMs of the device: the smallest split
    that keeps at least nine tenths of them busy, a function of the shape and the device alone
    (a result never depends on the batch)."""
    sms = sms if sms is not None else K.sm_count()
    tiles = -(-n_out // 128)
    k_tiles = -(-k // 64)
    best, best_fill = 1, 0.0
    for split in range(1, 9):
        if split > 1 and k_tiles // split < _MIN_K_TILES_PER_SPLIT:
            break
        blocks = tiles * split
        fill = blocks / (-(-blocks // sms) * sms)
        if fill > best_fill + 1e-9:
            best, best_fill = split, fill
        if fill >= 0.9:
            break
    return best


def _use_smallm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
                rows: int = _SMALLM_ROWS) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and out.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
            and x.shape[0] <= rows and x.shape[1] % 8 == 0
            and x.is_contiguous() and weight.is_contiguous() and out.is_contiguous())


def gated_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """out = silu(x Wg^T) * (x Wu^T) with weight = [Wg; Wu], in one kernel, where a hand-written
    kernel takes the case: the weight-streaming one up to 64 rows, the two-SM one (256 x 256
    tiles, persistent) above; False if the caller has to do it in steps.  At the 7B shape the
    two-SM kernel takes 55 / 93 / 352 us at 256 / 512 / 2048 rows, cuBLAS and the activation
    kernel behind it 76 / 101 / 392.  It also pays where its tiles do not fill the SM pairs: a decode
    step of the 0.5B shape at 256 rows (38 tiles of the 9728 x 896 weight) takes 1.53 ms with it and
    1.57 with the library and the activation kernel, although alone the library is ahead there
    (9.7 us against 11.9): inside a graph one launch less weighs more than the kernel's fixed cost."""
    if _use_smallm(x, weight, None, out, _GATED_ROWS):
        K.gemm_smallm_gated(x, weight, out)
        return True
    if _use_smallm(x, weight, None, out, 1 << 30) and K.gemm_large_gated_supported(
            x.shape[0], out.shape[1], x.shape[1]):
        K.gemm_large_gated(x, weight, out)
        return True
    return False



def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
           out: torch.Tensor, scratch=None) -> torch.Tensor:
    """out = x @ weight.T (+ bias).  x: [N, K], weight: [M, K], out: [N, M].  With few rows
    in bfloat16 the product runs on the hand-written tcgen05 kernel (`scratch` is the step's
    scratch allocator, for its split-K partials); otherwise in cuBLAS."""
    if scratch is not None and _use_smallm(x, weight, bias, out):
        m, k = x.shape
        n = weight.shape[0]
        K.gemm_smallm(x, weight, bias, out, ksplit=smallm_ksplit(m, n, k, K.sm_count(x.device)))
        return out
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
