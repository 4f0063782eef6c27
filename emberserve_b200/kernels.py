"""Python face of the hand-written CUDA kernels (``csrc/*.cu``), through ctypes.

Every function here takes CUDA tensors, checks what the kernel assumes (device,
contiguity, dtypes) and launches on the current torch stream.  There is no CPU path and
no library fallback: a missing or unbuildable extension, a tensor that is not on the
GPU, or a non-zero status from a launcher raises.

The launchers are plain ``extern "C"`` symbols taking raw pointers, so they are
captured by CUDA graphs like any other launch and allocate nothing themselves.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch

from emberserve_b200 import build

_ERRORS = {
    1: "unknown element type",
    2: "a size this kernel does not take",
    3: "the CUDA launch failed",
    4: "scratch buffer missing or too small",
    5: "pointer or stride not aligned as the kernel needs",
}


class KernelError(RuntimeError):
    pass


_lib_handle: ctypes.CDLL | None = None


def library() -> ctypes.CDLL:
    """The loaded extension; built on first use.  Raises if it cannot be had."""
    global _lib_handle
    if _lib_handle is None:
        path = build.ensure_built()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:  # pragma: no cover - depends on the machine
            raise KernelError(f"cannot load the emberserve_b200 CUDA extension {path}: {e}") from e
        _declare(lib)
        _lib_handle = lib
    return _lib_handle


def library_path() -> str:
    library()
    return str(build.ensure_built(verbose=False))


def _declare(lib: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "ems_embedding": [P, I, P, P, P, I, I, P],
        "ems_add_rmsnorm": [P, P, P, I, P, I, P, I, I, F, I, P],
        "ems_silu_mul": [P, P, I, I, I, P],
        "ems_rope_table": [P, P, I, I, P],
        "ems_rope_kv_write": [P, I, I, I, I, I, P, P, P, I, P, P, P, I, I, I, P],
        "ems_decode_attention_fused": [P, L, P, P, P, P, I, I, P, P, I, I, I, I, I, F, P, I, I, I, P, L, P],
        "ems_paged_attention": [P, L, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, F, I, I, P, L, I, P],
        "ems_argmax": [P, P, I, I, P, P],
        "ems_repetition_penalty": [P, I, I, P, P, P, P],
        "ems_sample": [P, I, I, P, P, P, P, P, P, P],
        "ems_gemm_smallm": [P, P, P, P, I, I, I, I, P, P, P, P, P, I, I, F, I, I, P],
        "ems_gemm_smallm_gated": [P, P, P, I, I, I, P, I, I, F, I, P],
        "ems_gemm_midm": [P, P, P, P, I, I, I, I, I, P],
        "ems_gemm_midm_max_clusters": [I, I],
        "ems_gemm_large_gated": [P, P, P, I, I, I, I, P],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    lib.ems_gemm_large_gated_supported.argtypes = [I, I, I]
    lib.ems_gemm_large_gated_supported.restype = c_int
    lib.ems_gemm_smallm_status.argtypes = []
    lib.ems_gemm_smallm_status.restype = c_int
    lib.ems_tc_status_clear.argtypes = []
    lib.ems_tc_status_clear.restype = None
    lib.ems_argmax_slices.argtypes = [I, I]
    lib.ems_argmax_slices.restype = c_int
    lib.ems_paged_attention_scratch_bytes.argtypes = [I, I, I, I]
    lib.ems_paged_attention_scratch_bytes.restype = c_longlong


_sm_counts: dict[int, int] = {}
# What a helper assumes where there is no device to ask (the host-logic tests): a B200.
B200_SMS = 148


def sm_count(device: "torch.device | str | None" = None) -> int:
    """Streaming multiprocessors of `device` (asked once per device); the grid-shaping helpers
    (how keys or K are split over blocks) take it from here instead of a constant."""
    dev = torch.device(device) if device is not None else None
    if dev is not None and dev.type != "cuda":
        return B200_SMS
    key = dev.index if dev is not None and dev.index is not None else -1
    n = _sm_counts.get(key)
    if n is None:
        # (the driver is asked here only: a question about the device count at every call is slow
        # and can wait behind other users of the driver)
        if not torch.cuda.is_available():
            return B200_SMS
        idx = key if key >= 0 else torch.cuda.current_device()
        n = _sm_counts[key] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (eager launches; a CUDA
    graph replay adds what its capture recorded)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'status {code}')}")
    _launches += kernels


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: torch.Tensor | None, name: str = "tensor") -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (emberserve_b200 has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t.data_ptr()


def _i32(t: torch.Tensor | None, name: str) -> int | None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    return _ptr(t, name)


def _stream() -> int:
    # the raw handle of torch's current stream (the capturing stream inside a graph capture);
    # the public torch.cuda.current_stream() costs tens of microseconds per call
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_stream_objects: dict[tuple[int, int], "torch.cuda.Stream"] = {}


def record_event() -> "torch.cuda.Event":
    """A new event recorded on the current stream.  The stream object is looked up by its raw
    handle and kept: ``torch.cuda.current_stream()`` asks the driver for the device count at every
    call, which is slow and can stall behind other users of the driver."""
    key = (torch._C._cuda_getDevice(), _stream())
    stream = _stream_objects.get(key)
    if stream is None:
        stream = _stream_objects[key] = torch.cuda.current_stream()
    event = torch.cuda.Event()
    event.record(stream)
    return event


# ---------------------------------------------------------------------------------------


def embedding(table: torch.Tensor, tokens: torch.Tensor, residual: torch.Tensor,
              deferred: torch.Tensor | None = None) -> None:
    """residual[n, :] = float32(table[tokens[n], :]); a token -(k + 1) reads deferred[k] (a token
    sampled on the device by an earlier kernel of the stream)."""
    n, h = residual.shape
    assert table.shape[1] == h and residual.dtype == torch.float32 and tokens.numel() >= n
    _check(library().ems_embedding(_ptr(table, "table"), _dt(table), _i32(tokens, "tokens"),
                                   None if deferred is None else _i32(deferred, "deferred"),
                                   _ptr(residual, "residual"), n, h, _stream()), "embedding")


def add_rmsnorm(delta: torch.Tensor | None, residual: torch.Tensor, weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
                num_rows: int | None = None) -> None:
    """residual += delta (32-bit); out = weight * round(residual * rsqrt(mean(residual^2) + eps)).
    With `rows`, only residual rows rows[0..num_rows) are normalised into out[0..num_rows)
    and the residual is not written."""
    h = residual.shape[-1]
    assert residual.dtype == torch.float32 and weight.numel() == h and out.shape[-1] == h
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape[-1] == h
    n_out = residual.shape[0] if rows is None else (rows.numel() if num_rows is None else num_rows)
    if delta is not None and rows is None:
        assert delta.shape[0] >= n_out
    _check(library().ems_add_rmsnorm(_ptr(delta, "delta"), _ptr(residual, "residual"),
                                     _ptr(weight, "weight"), _dt(weight), _ptr(out, "out"), _dt(out),
                                     _i32(rows, "rows"), n_out, h, float(eps),
                                     0 if rows is not None else 1, _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]"""
    n, i = out.shape
    assert gate_up.shape == (n, 2 * i) and gate_up.dtype == out.dtype
    _check(library().ems_silu_mul(_ptr(gate_up, "gate_up"), _ptr(out, "out"), _dt(out), n, i,
                                  _stream()), "silu_mul")


def rope_table(inv_freq: torch.Tensor, max_pos: int) -> torch.Tensor:
    """[max_pos, half, 2] float32 table of (cos, sin) of pos * inv_freq[i], both 32-bit."""
    assert inv_freq.dtype == torch.float32
    half = inv_freq.numel()
    table = torch.empty(max_pos, half, 2, dtype=torch.float32, device=inv_freq.device)
    _check(library().ems_rope_table(_ptr(inv_freq, "inv_freq"), _ptr(table), max_pos, half,
                                    _stream()), "rope_table")
    return table


def rope_kv_write(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                  positions: torch.Tensor, row_of_token: torch.Tensor,
                  table: torch.Tensor | None, rotary_dim: int,
                  kcache: torch.Tensor | None, vcache: torch.Tensor | None,
                  block_tables: torch.Tensor | None, page_size: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k by the table rows of `positions`; store k and v of every
    token at its page slot.  qkv: [N, (nh + 2 nkv) D]; caches [pages, nkv, page_size, D]."""
    n = qkv.shape[0]
    assert qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    if write_kv:
        assert kcache is not None and vcache is not None and block_tables is not None
        assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype
        assert kcache.shape[1:] == (num_kv_heads, page_size, head_dim)
    bt_stride = block_tables.shape[1] if block_tables is not None else 0
    _check(library().ems_rope_kv_write(
        _ptr(qkv, "qkv"), _dt(qkv), n, num_heads, num_kv_heads, head_dim,
        _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _ptr(table, "table"),
        rotary_dim, _ptr(kcache, "kcache"), _ptr(vcache, "vcache"),
        _i32(block_tables, "block_tables"), bt_stride, page_size, 1 if write_kv else 0, _stream()),
        "rope_kv_write")


def attention_scratch_bytes(num_tokens: int, num_heads: int, head_dim: int, splits: int) -> int:
    return int(library().ems_paged_attention_scratch_bytes(num_tokens, num_heads, head_dim, splits))


_ATTENTION_IMPL = {"auto": 0, "generic": 1, "tcgen05": 2, "mma": 3}


def paged_attention(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    block_tables: torch.Tensor, cu_q: torch.Tensor, starts: torch.Tensor,
                    num_rows: int, num_tokens: int, num_heads: int, num_kv_heads: int,
                    head_dim: int, scale: float, max_q_len: int, window: int | None = None,
                    splits: int = 1, scratch: torch.Tensor | None = None, generic: bool = False,
                    tcgen05: bool = False, kernel: str = "auto") -> None:
    """Causal grouped-query attention of every packed query over its request's pages.
    `q` is a [N, stride] tensor whose first nh*D columns are the queries (a view of the
    qkv buffer is fine); `out` is [N, nh*D].  `generic=True` forces the generic kernel where
    a faster one would take the case (tests compare the two); `tcgen05=True` asks for the
    tcgen05 prompt kernel at any length (by default it takes the long portions) and raises if
    that kernel does not take the case.  `kernel` says the same by name: "auto", "generic",
    "tcgen05", or "mma" (the mma.sync kernels where they take the case)."""
    assert q.stride(1) == 1 and out.is_contiguous() and q.dtype == out.dtype == kcache.dtype
    page_size = kcache.shape[2]
    assert kcache.shape[1] == num_kv_heads and kcache.shape[3] == head_dim
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_paged_attention(
        q.data_ptr(), q.stride(0), _ptr(out, "out"), _dt(out), _ptr(kcache, "kcache"),
        _ptr(vcache, "vcache"), _i32(block_tables, "block_tables"), block_tables.shape[1], page_size,
        _i32(cu_q, "cu_q"), _i32(starts, "starts"), num_rows, num_tokens, num_heads, num_kv_heads,
        head_dim, int(window or 0), float(scale), max_q_len, splits,
        _ptr(scratch, "scratch"), 0 if scratch is None else scratch.numel() * scratch.element_size(),
        _ATTENTION_IMPL["generic" if generic else ("tcgen05" if tcgen05 else kernel)], _stream()),
        "paged_attention", 2 if splits > 1 else 1)


def decode_attention_fused_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                                     rotary_dim: int) -> bool:
    """Whether `decode_attention_fused` takes the geometry (the alignment of the tensors is
    checked by the call itself)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads // num_kv_heads <= 16
            and rotary_dim in (0, head_dim))


def decode_attention_fused(qkv: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                           block_tables: torch.Tensor, cu_q: torch.Tensor, starts: torch.Tensor, num_rows: int,
                           num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                           rope_table: torch.Tensor | None, rotary_dim: int, write_kv: bool,
                           window: int | None = None, splits: int = 1, scratch: torch.Tensor | None = None) -> None:
    """A decode step's attention (every row brings one token) with the rotary encoding of q and
    k and the write of the new key and value done by the attention kernel itself: `qkv` holds
    the raw projections [q | k | v].  With `splits` > 1, `scratch` takes the partials and the merge
    kernel follows."""
    assert qkv.stride(1) == 1 and out.is_contiguous() and qkv.dtype == out.dtype == kcache.dtype == torch.bfloat16
    assert rope_table is None or rope_table.dtype == torch.float32
    _check(library().ems_decode_attention_fused(
        qkv.data_ptr(), qkv.stride(0), _ptr(out, "out"), _ptr(kcache, "kcache"), _ptr(vcache, "vcache"),
        _i32(block_tables, "block_tables"), block_tables.shape[1], kcache.shape[2], _i32(cu_q, "cu_q"),
        _i32(starts, "starts"), num_rows, num_heads, num_kv_heads, head_dim, int(window or 0), float(scale),
        _ptr(rope_table, "rope_table"), rotary_dim, 1 if write_kv else 0, splits, _ptr(scratch, "scratch"),
        0 if scratch is None else scratch.numel() * scratch.element_size(), _stream()),
        "decode_attention_fused", 2 if splits > 1 else 1)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the maximum of logits[r]."""
    r, v = logits.shape
    assert logits.dtype == torch.float32
    slices = library().ems_argmax_slices(r, v)
    tmp = torch.empty(r * slices, dtype=torch.int64, device=logits.device) if slices else None
    _check(library().ems_argmax(_ptr(logits, "logits"), _i32(out, "out"), r, v, _ptr(tmp, "tmp"), _stream()),
           "argmax", 2 if slices else 1)


def repetition_penalty(logits: torch.Tensor, row_ptr: torch.Tensor, token_ids: torch.Tensor,
                       penalty: torch.Tensor) -> None:
    r, v = logits.shape
    assert logits.dtype == torch.float32 and penalty.dtype == torch.float32
    _check(library().ems_repetition_penalty(_ptr(logits, "logits"), r, v, _i32(row_ptr, "row_ptr"),
                                            _i32(token_ids, "token_ids"), _ptr(penalty, "penalty"),
                                            _stream()), "repetition_penalty")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: torch.Tensor) -> None:
    """One token per row: argmax where temperature == 0, else a seeded draw."""
    r, v = logits.shape
    assert logits.dtype == torch.float32 and temperature.dtype == torch.float32
    assert top_p.dtype == torch.float32 and seeds.dtype == torch.int64 and counters.dtype == torch.int64
    _check(library().ems_sample(_ptr(logits, "logits"), r, v, _ptr(temperature, "temperature"),
                                _i32(top_k, "top_k"), _ptr(top_p, "top_p"), _ptr(seeds, "seeds"),
                                _ptr(counters, "counters"), _i32(out, "out"), _stream()), "sample")


GEMM_SMALLM_MAX_ROWS = 64


# Rows of a step up to which the small-row products can take a norm into their epilogues.
GEMM_NORM_ROWS = 16


@dataclass
class NormBehind:
    """The norm that stands behind a small-row product, begun in the product's epilogue: the
    product is added into `residual` (float32 [m, n], in place) instead of being stored,
    `scaled` (bfloat16 [m, n]) receives residual * gain, and `sumsq` (float32 [parts, 16],
    parts = row tiles * ksplit of the product) every block's share of each row's sum of squares."""

    residual: torch.Tensor
    gain: torch.Tensor
    scaled: torch.Tensor
    sumsq: torch.Tensor


@dataclass
class NormBefore:
    """The norm that stands before a small-row product, finished in its epilogue: the product
    was given residual * gain, and row n of its result is multiplied by
    1 / sqrt(sumsq[:parts, n].sum() / width + eps) before the bias is added."""

    sumsq: torch.Tensor
    parts: int
    width: int
    eps: float


def _norm_before_args(nb: "NormBefore | None", m: int) -> tuple:
    if nb is None:
        return (None, 0, 0, 0.0)
    assert nb.sumsq.dtype == torch.float32 and nb.sumsq.numel() >= nb.parts * GEMM_NORM_ROWS and m <= GEMM_NORM_ROWS
    return (_ptr(nb.sumsq, "sumsq"), nb.parts, nb.width, float(nb.eps))


def tile_weight_shape_ok(weight: torch.Tensor) -> bool:
    """Whether `tile_weight` has a tiled form for this weight."""
    return (weight.dim() == 2 and weight.dtype == torch.bfloat16 and weight.is_cuda and weight.is_contiguous()
            and weight.shape[0] % 128 == 0 and weight.shape[1] % 64 == 0)


def tile_weight(weight: torch.Tensor) -> torch.Tensor | None:
    """The tiled copy of a bfloat16 weight [n, k] that the weight-streaming kernels read faster: the
    128 x 64 tile (row tile r, K tile kt) as 16 KB of contiguous memory at tile index
    r * (k / 64) + kt, so that one TMA load reads whole DRAM pages instead of 128 bytes from each of
    128 rows (7B shape: gate / up product 45.1 -> 43.9 us, down 25.2 -> 24.5, the decode step at
    batch 8 2.90 -> 2.82 ms).  None where n or k is no multiple of 128 / 64.  The copy has the
    shape [n * k / 64, 64]; it is passed as `twin` beside the weight it was made of."""
    if not tile_weight_shape_ok(weight):
        return None
    n, k = weight.shape
    return weight.view(n // 128, 128, k // 64, 64).permute(0, 2, 1, 3).contiguous().view(n * (k // 64), 64)


def _weight_ptr(weight: torch.Tensor, twin: torch.Tensor | None) -> tuple[int | None, int]:
    if twin is None:
        return _ptr(weight, "weight"), 0
    n, k = weight.shape
    assert twin.dtype == weight.dtype and twin.shape == (n * (k // 64), 64) and n % 128 == 0 and k % 64 == 0
    assert twin.is_contiguous()
    return _ptr(twin, "twin"), 1


def gemm_smallm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor | None,
                ksplit: int = 1, norm_behind: NormBehind | None = None,
                norm_before: NormBefore | None = None, twin: torch.Tensor | None = None) -> None:
    """out[m, n] = x[m, :] . weight[n, :] (+ bias[n]) in bfloat16 with float32 accumulation, for
    m <= 64 rows: the weight-streaming tcgen05 kernel.  `ksplit` blocks (up to 8) share K: they
    form a thread-block cluster and add their accumulators on chip, in rank order.  With
    `norm_behind` the product joins the residual stream in the epilogue (`out` is not written and
    may be None); with `norm_before` its rows are scaled there (m <= 16 for both)."""
    m, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k and (out is None or out.shape == (m, n))
    assert x.dtype == weight.dtype == torch.bfloat16
    # (a float32 `out` takes the sums unrounded: only where one block holds the whole sum)
    f32 = out is not None and out.dtype == torch.float32
    assert out is None or out.dtype == torch.bfloat16 or (f32 and ksplit == 1 and norm_behind is None)
    assert bias is None or (bias.dtype == torch.bfloat16 and bias.numel() == n)
    behind = (None, None, None, None)
    if norm_behind is not None:
        nb = norm_behind
        parts = -(-n // 128) * ksplit
        assert m <= GEMM_NORM_ROWS and nb.residual.dtype == torch.float32 and nb.residual.shape == (m, n)
        assert nb.gain.dtype == torch.bfloat16 and nb.gain.numel() == n
        assert nb.scaled.dtype == torch.bfloat16 and nb.scaled.shape == (m, n)
        assert nb.sumsq.dtype == torch.float32 and nb.sumsq.numel() >= parts * GEMM_NORM_ROWS
        behind = (_ptr(nb.residual, "residual"), _ptr(nb.gain, "gain"), _ptr(nb.scaled, "scaled"),
                  _ptr(nb.sumsq, "sumsq"))
    else:
        assert out is not None
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_smallm(
        _ptr(x, "x"), wptr, _ptr(bias, "bias"), _ptr(out, "out"), m, n, k, ksplit,
        *behind, *_norm_before_args(norm_before, m), tiled, 1 if f32 else 0, _stream()), "gemm_smallm")


GEMM_MIDM_ROWS = 128
_midm_clusters: dict[tuple[int, int, int], int] = {}


def gemm_midm_max_clusters(m: int, ksplit: int, device: "torch.device | None" = None) -> int:
    """How many clusters of `ksplit` blocks of the kernel for `m` rows (one block per SM) the device
    holds at once; a cluster lives inside one of the GPU's processing clusters, so this is less than
    SMs // ksplit (a B200 holds 148, 74, 45, 33, 26, 22, 15, 15 for 1..8).  Asked once per size."""
    nt = 32 if m <= 32 else (64 if m <= 64 else 128)
    idx = -1 if device is None or device.index is None else device.index
    key = (idx, nt, ksplit)
    n = _midm_clusters.get(key)
    if n is None:
        n = int(library().ems_gemm_midm_max_clusters(nt, ksplit))
        if n < 0:
            raise KernelError(f"gemm_midm: the occupancy of clusters of {ksplit} could not be asked")
        _midm_clusters[key] = n
    return n


def gemm_midm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
              ksplit: int = 1, twin: torch.Tensor | None = None) -> None:
    """out[m, n] = x[m, k] @ weight[n, k].T (+ bias) in bfloat16 for up to 128 rows: the tcgen05
    kernel with one block per SM and a deep ring.  `ksplit` (1..8) blocks share K as a cluster;
    the caller picks it so that all blocks start in one wave."""
    m, k = x.shape
    n = weight.shape[0]
    assert x.dtype == weight.dtype == out.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
    assert x.is_contiguous() and weight.is_contiguous() and out.is_contiguous()
    assert weight.shape[1] == k and out.shape == (m, n)
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_midm(_ptr(x, "x"), wptr, _ptr(bias, "bias"), _ptr(out, "out"),
                                   m, n, k, ksplit, tiled, _stream()), "gemm_midm")


def gemm_smallm_gated(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                      norm_before: NormBefore | None = None, twin: torch.Tensor | None = None) -> None:
    """out[m, i] = silu(x . weight[i]) * (x . weight[I + i]) for weight [2 I, K]: gate and up
    projections of a gated feed-forward and its activation in one tcgen05 kernel, m <= 64.  With
    `norm_before` (m <= 16) both projections' rows are scaled first, as in `gemm_smallm`."""
    m, k = x.shape
    inter = out.shape[1]
    assert weight.shape == (2 * inter, k) and out.shape[0] == m
    assert x.dtype == weight.dtype == out.dtype == torch.bfloat16
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_smallm_gated(_ptr(x, "x"), wptr, _ptr(out, "out"), m, inter, k,
                                           *_norm_before_args(norm_before, m), tiled, _stream()), "gemm_smallm_gated")


def gemm_large_gated_supported(m: int, inter: int, k: int) -> bool:
    """Whether gemm_large_gated takes these sizes (bfloat16 tensors)."""
    return bool(library().ems_gemm_large_gated_supported(m, inter, k))


def gemm_large_gated(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                     twin: torch.Tensor | None = None) -> None:
    """out[m, i] = silu(x . weight[i]) * (x . weight[I + i]) for weight [2 I, K] and any number
    of rows m: the two-SM tcgen05 kernel of prompt steps (256 x 256 tiles, persistent grid), with
    the activation in its epilogue.  I a multiple of 128, K a multiple of 8."""
    m, k = x.shape
    inter = out.shape[1]
    assert weight.shape == (2 * inter, k) and out.shape[0] == m
    assert x.dtype == weight.dtype == out.dtype == torch.bfloat16
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_large_gated(_ptr(x, "x"), wptr, _ptr(out, "out"), m, inter, k, tiled,
                                          _stream()), "gemm_large_gated")


def gemm_smallm_status() -> int:
    """0, or the code of the first bounded wait that ran out in the tcgen05 kernel (after a
    synchronisation point): 1 producer, 2 MMA issuer, 3 epilogue, 4 drain, 5 arrival of the split-K
    partials of the small-row kernel;
    11 producer, 12 and 13 MMA issuer, 14 epilogue of the two-SM kernel; 31 producer, 32 MMA issuer,
    33 epilogue, 34 drain, 35 arrival of the partials of the kernel for 17..128 rows; 20 and up: the
    prompt attention."""
    return int(library().ems_gemm_smallm_status())


def clear_status() -> None:
    """Set the status word of the tcgen05 kernels back to 0 (after the device has been waited for)."""
    library().ems_tc_status_clear()


def check_status(clear: bool = True) -> None:
    """Raise if a bounded wait inside a tcgen05 kernel (a GEMM or the prompt attention) ran out
    since the word was last cleared: what that kernel wrote is invalid, and so is everything
    computed from it.  The word lives in host-mapped memory, so the check costs no CUDA call; it
    means something only after a synchronisation point behind the kernels in question.  With
    `clear` the word is reset, so that the next step starts clean."""
    code = gemm_smallm_status()
    if code != 0:
        if clear:
            clear_status()
        raise KernelError(f"a wait inside a tcgen05 kernel ran out (code {code}); the results of the "
                          f"step are invalid")
