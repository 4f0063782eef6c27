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
from emberserve_b200.parts.base import NormRequest, ScaledRows


def strict_matmul_precision() -> None:
    """Process-wide matmul settings of the engine: no TF32, no split-K in bfloat16."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


_MIN_K_TILES_PER_SPLIT = 4
_MAX_KSPLIT = 8  # the portable size of a thread-block cluster
# Up to this many rows the hand-written kernel is used; with more, cuBLAS is as fast or faster
# (measured at the projection shapes of a 7B model).
_SMALLM_ROWS = 16
# The gate/up product with SiLU in its epilogue stays ahead up to the kernel's 64 rows: cuBLAS
# needs a separate activation kernel behind it (decode step of the 7B shape at 24 / 32 / 64 rows:
# 4.05 / 4.37 / 5.51 ms against 4.25 / 4.48 / 5.65).
_GATED_ROWS = 64


def smallm_ksplit(m_tok: int, n_out: int, k: int, sms: int | None = None) -> int:
    """Over how many blocks (one thread-block cluster, at most 8) the small-row kernel splits K:
    the LARGEST split whose blocks all start at once on the `sms` SMs of the device.  These
    products are chains of short waits (fill the ring, multiply, push the partial sums, store)
    as much as streams, so the shortest K range per block wins as long as no cluster has to wait
    for a second wave; a K range keeps at least four 64-column tiles.  Two blocks share an SM, but
    a cluster has to fit into one of the GPU's processing clusters, so not every slot can be
    filled: 6/7 of them is what starts in one wave on a B200 (36 clusters of 7 do, 36 of 8 do
    not).  A function of the shape and the device alone: a result never depends on the batch."""
    sms = sms if sms is not None else K.sm_count()
    tiles = -(-n_out // 128)
    k_tiles = -(-k // 64)
    slots = (2 * sms * 6) // 7
    best = 1
    for split in range(2, _MAX_KSPLIT + 1):
        if k_tiles // split < _MIN_K_TILES_PER_SPLIT:
            break
        if tiles * split <= slots:
            best = split
    return best


def tiled_twin(weight: torch.Tensor) -> torch.Tensor | None:
    """The tiled copy of `weight` for the weight-streaming kernels, if the engine made one
    (`give_tiled_twin`)."""
    return getattr(weight, "tiled_twin", None)


def give_tiled_twin(weight: torch.Tensor) -> int:
    """Make the tiled copy of a weight that decode steps stream (`kernels.tile_weight`) and hang it
    on the tensor; the bytes it takes (0 where the shape has none)."""
    twin = K.tile_weight(weight)
    if twin is None:
        return 0
    weight.tiled_twin = twin
    return twin.numel() * twin.element_size()


def midm_ksplit(m_tok: int, n_out: int, k: int, clusters=None) -> int:
    """Over how many blocks (one cluster, at most 8) the kernel for 17..128 rows splits K: it keeps
    one block per SM, so the largest split of which the device holds as many clusters at once as
    the product has 128-row tiles (`clusters(split)`, by default asked from the device); a K range
    keeps at least two 64-column tiles.  A function of the shape and the device alone."""
    clusters = clusters or (lambda split: K.gemm_midm_max_clusters(m_tok, split))
    tiles = -(-n_out // 128)
    k_tiles = -(-k // 64)
    best = 1
    for split in range(2, _MAX_KSPLIT + 1):
        if k_tiles // split < 2:
            break
        if tiles <= clusters(split):
            best = split
    return best


def _use_midm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> int:
    """The K split with which the tcgen05 kernel for 17..128 rows takes the product, or 0 where
    cuBLAS stays.  It takes products with a long K and few output tiles (K >= 2 N: the down
    projection of a gated feed-forward), where the library does not split K well: 7B shape
    (3584 x 18944) 27.0 / 28.6 / 31.7 us at 17 / 64 / 96 rows (25.8 / 27.8 / 30.9 from the tiled copy
    of the weight) against 31.7 / 32.1 / 32.7, 0.5B
    shape (896 x 4864) 4.8 / 6.4 against 8.7 / 8.4 at 17 / 64.  At squarer shapes (qkv, o) its fixed
    cost (set-up, and the partial sums of up to 64 KB per block that cross the cluster) leaves it
    0.3..2.6 us behind the library's 8..9 us, and from 97 rows on the activation tiles, as large as
    the weight tiles, take the SMs' inbound bandwidth."""
    m, k = x.shape
    n = weight.shape[0]
    if not (_SMALLM_ROWS < m <= 96 and k >= 2 * n and _use_smallm(x, weight, bias, out, 96)):
        return 0
    ksplit = midm_ksplit(m, n, k)
    if m > 64 and -(-k // 64) // ksplit < 32:
        return 0
    return ksplit


def _use_smallm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
                rows: int = _SMALLM_ROWS) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and out.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
            and x.shape[0] <= rows and x.shape[1] % 8 == 0
            and x.is_contiguous() and weight.is_contiguous() and out.is_contiguous())


def _norm_before(x: ScaledRows) -> K.NormBefore:
    return K.NormBefore(x.sumsq, x.parts, x.x.shape[1], x.eps)


def gated_linear(x: "torch.Tensor | ScaledRows", weight: torch.Tensor, out: torch.Tensor) -> bool:
    """out = silu(x Wg^T) * (x Wu^T) with weight = [Wg; Wu], in one kernel, where a hand-written
    kernel takes the case: the weight-streaming one up to 64 rows, the two-SM one (256 x 256
    tiles, persistent) above; False if the caller has to do it in steps.  At the 7B shape the
    two-SM kernel takes 55 / 93 / 352 us at 256 / 512 / 2048 rows, cuBLAS and the activation
    kernel behind it 76 / 101 / 392.  It also pays where its tiles do not fill the SM pairs: a decode
    step of the 0.5B shape at 256 rows (38 tiles of the 9728 x 896 weight) takes 1.53 ms with it and
    1.57 with the library and the activation kernel, although alone the library is ahead there
    (9.7 us against 11.9): inside a graph one launch less weighs more than the kernel's fixed cost."""
    if isinstance(x, ScaledRows):  # a norm that this product has to finish
        if _use_smallm(x.x, weight, None, out, K.GEMM_NORM_ROWS):
            K.gemm_smallm_gated(x.x, weight, out, norm_before=_norm_before(x), twin=tiled_twin(weight))
            return True
        x = x.materialize()
    if _use_smallm(x, weight, None, out, _GATED_ROWS):
        K.gemm_smallm_gated(x, weight, out, twin=tiled_twin(weight))
        return True
    if _use_smallm(x, weight, None, out, 1 << 30) and K.gemm_large_gated_supported(
            x.shape[0], out.shape[1], x.shape[1]):
        # (one tile of token rows streams the weight once, and the tiled copy streams faster: 56.1 ->
        # 53.6 us at 256 rows of the 7B shape; with more row tiles the weight is re-read from L2,
        # where the copy is no help and at 2048 rows a loss: 355 -> 405 us)
        K.gemm_large_gated(x, weight, out, twin=tiled_twin(weight) if x.shape[0] <= 256 else None)
        return True
    return False



def linear(x: "torch.Tensor | ScaledRows", weight: torch.Tensor, bias: torch.Tensor | None,
           out: torch.Tensor, scratch=None, behind: NormRequest | None = None) -> "torch.Tensor | ScaledRows":
    """out = x @ weight.T (+ bias).  x: [N, K], weight: [M, K], out: [N, M].  With few rows
    in bfloat16 the product runs on the hand-written tcgen05 kernel (`scratch` is the step's
    scratch allocator); otherwise in cuBLAS.

    `x` may be `ScaledRows`, the input of a norm still to be finished: the kernel scales the
    rows of the product (or the norm is finished the plain way first).  With `behind`, a
    `NormRequest`, the kernel adds the product into the residual stream, begins that norm and
    `ScaledRows` come back instead of `out` (which is then not written); where the kernel does
    not take the case the request is ignored and `out` comes back as always."""
    before = None
    if isinstance(x, ScaledRows):
        if scratch is not None and _use_smallm(x.x, weight, bias, out, K.GEMM_NORM_ROWS):
            before, x = _norm_before(x), x.x
        else:
            x = x.materialize()
    if scratch is not None and _use_smallm(x, weight, bias, out):
        m, k = x.shape
        n = weight.shape[0]
        ksplit = smallm_ksplit(m, n, k, K.sm_count(x.device))
        if (behind is not None and m <= K.GEMM_NORM_ROWS and behind.residual.shape == (m, n)
                and behind.gain.dtype == torch.bfloat16):
            parts = -(-n // 128) * ksplit
            rows = ScaledRows(scratch("normed", (m, n), torch.bfloat16),
                              scratch("norm_sumsq", (parts, K.GEMM_NORM_ROWS), torch.float32), parts, behind.eps)
            K.gemm_smallm(x, weight, bias, None, ksplit=ksplit, norm_before=before, twin=tiled_twin(weight),
                          norm_behind=K.NormBehind(behind.residual, behind.gain, rows.x, rows.sumsq))
            return rows
        K.gemm_smallm(x, weight, bias, out, ksplit=ksplit, norm_before=before, twin=tiled_twin(weight))
        return out
    if scratch is not None:
        ksplit = _use_midm(x, weight, bias, out)
        if ksplit:
            K.gemm_midm(x, weight, bias, out, ksplit=ksplit, twin=tiled_twin(weight))
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
    if (x.is_cuda and x.dtype == weight.dtype == torch.bfloat16 and out.dtype == torch.float32
            and x.shape[0] <= _SMALLM_ROWS and x.shape[1] % 8 == 0
            and x.is_contiguous() and weight.is_contiguous() and out.is_contiguous()):
        # few rows: the weight-streaming kernel, one block per 128 outputs (no K split: the sum is
        # stored unrounded by the block that holds it).  7B shape (152064 x 3584), 8 rows: 157 us
        # from the tiled copy, 160 from the row-major matrix, cuBLAS 182.
        K.gemm_smallm(x, weight, None, out, ksplit=1, twin=tiled_twin(weight))
        return out
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
