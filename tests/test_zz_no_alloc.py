"""The entry point that allocates nothing, ``ems_paged_attention_static_scratch``, called
through its exported C symbol, against the ordinary entry point with a scratch buffer
that torch allocated.

Who this is for: a program that cannot call cudaMalloc where it calls the kernel (all GPU
memory already belongs to its own pool, or allocation is forbidden on its hot path because
it synchronises the device, or it is plain C with no tensor library).  Such a caller
passes inputs and outputs only; the partial results of the key splits go to a fixed 8 MiB
array inside the library.  The file is named so that pytest collects it last: a run that
stops at the first failure has then already run every other test.
"""

from __future__ import annotations

import ctypes
import gc
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _symbol():
    from emberserve_b200 import kernels

    lib = kernels.library()
    fn = lib.ems_paged_attention_static_scratch
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    fn.argtypes = [P, L, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, F, I, I, P]
    fn.restype = c_int
    lib.ems_static_scratch_capacity.argtypes = []
    lib.ems_static_scratch_capacity.restype = c_longlong
    return lib, fn


def _case(seed, dtype, b, nh, nkv, d, ps, max_ctx):
    g = torch.Generator(device="cuda").manual_seed(seed)
    starts = torch.randint(0, max_ctx, (b,), generator=g, device=DEV).to(torch.int32)
    width = max_ctx // ps + 2
    pages = b * width
    bt = torch.randperm(pages, device=DEV, generator=g).view(b, width).to(torch.int32)
    kc = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(dtype)
    vc = torch.randn(pages, nkv, ps, d, device=DEV, generator=g).to(dtype)
    qkv = (torch.randn(b, (nh + 2 * nkv) * d, device=DEV, generator=g) * 2).to(dtype)
    cu = torch.arange(b + 1, device=DEV, dtype=torch.int32)
    return qkv, kc, vc, bt, cu, starts


def _call(fn, qkv, out, kc, vc, bt, cu, starts, rows, tokens, nh, nkv, d, window, max_q_len, splits):
    return fn(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), 0 if out.dtype == torch.float32 else 1,
              kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.shape[1], kc.shape[2], cu.data_ptr(),
              starts.data_ptr(), rows, tokens, nh, nkv, d, window, 1 / math.sqrt(d), max_q_len, splits,
              torch.cuda.current_stream().cuda_stream)


# (rows, heads, KV heads, head size, page size, splits): the mma.sync decode kernel at both of its
# head sizes, and a head size that only the generic kernel takes
GEOMETRIES = [(6, 28, 4, 128, 16, 8), (5, 14, 2, 64, 16, 6), (4, 6, 2, 48, 8, 5)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("geometry", GEOMETRIES, ids=["d128", "d64", "d48"])
def test_static_scratch_entry_equals_the_allocating_one_twice_in_a_row(dtype, geometry):
    """Two calls in a row (the second finds what the first left in the array) give, bit for bit,
    what the ordinary entry point gives with a scratch buffer of the caller's: they run the same
    kernels over the same splits.  Neither torch's allocator nor the device's free memory moves
    across the call."""
    from emberserve_b200 import kernels as K

    lib, fn = _symbol()
    b, nh, nkv, d, ps, splits = geometry
    assert K.attention_scratch_bytes(b, nh, d, splits) <= lib.ems_static_scratch_capacity()
    for call, (seed, max_ctx, window) in enumerate([(1, 900, 0), (2, 300, 70)]):
        qkv, kc, vc, bt, cu, starts = _case(seed, dtype, b, nh, nkv, d, ps, max_ctx)
        want = torch.empty(b, nh * d, dtype=dtype, device=DEV)
        scratch = torch.empty(K.attention_scratch_bytes(b, nh, d, splits) // 4, device=DEV)
        K.paged_attention(qkv, want, kc, vc, bt, cu, starts, b, b, nh, nkv, d, 1 / math.sqrt(d), 1,
                          window=window or None, splits=splits, scratch=scratch, kernel="mma")
        got = torch.full_like(want, float("nan"))
        if call == 0:  # the first call on the device takes the array's address; not counted below
            assert _call(fn, qkv, got, kc, vc, bt, cu, starts, b, b, nh, nkv, d, window, 1, splits) == 0
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        # (what earlier tests left behind in reference cycles is collected now, not during the call,
        # where it would move torch's counter)
        gc.collect()
        gc.disable()
        try:
            before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info(DEV)[0]
            rc = _call(fn, qkv, got, kc, vc, bt, cu, starts, b, b, nh, nkv, d, window, 1, splits)
            torch.cuda.synchronize()
            after, free_after = torch.cuda.memory_allocated(), torch.cuda.mem_get_info(DEV)[0]
        finally:
            gc.enable()
        assert rc == 0, f"call {call}: status {rc}"
        assert after == before, "the call moved torch's allocator"
        assert free_after == free_before, "the call changed the device's free memory"
        assert torch.equal(got, want), f"call {call}: {(got.float() - want.float()).abs().max()}"


def test_static_scratch_entry_without_splits_takes_prompt_portions():
    """splits == 1 needs no scratch: the call is handed on to the ordinary entry point (never to
    the tcgen05 kernel, whose first use allocates), here with rows of several tokens."""
    from emberserve_b200 import kernels as K

    lib, fn = _symbol()
    nh, nkv, d, ps = 8, 2, 64, 16
    q_lens, cached = [5, 1, 37], [40, 100, 0]
    b, n = len(q_lens), sum(q_lens)
    g = torch.Generator(device="cuda").manual_seed(11)
    width = 12
    bt = torch.randperm(b * width, device=DEV, generator=g).view(b, width).to(torch.int32)
    kc = torch.randn(b * width, nkv, ps, d, device=DEV, generator=g).bfloat16()
    vc = torch.randn(b * width, nkv, ps, d, device=DEV, generator=g).bfloat16()
    qkv = torch.randn(n, (nh + 2 * nkv) * d, device=DEV, generator=g).bfloat16()
    cu = torch.tensor([0, 5, 6, 43], dtype=torch.int32, device=DEV)
    starts = torch.tensor(cached, dtype=torch.int32, device=DEV)
    want = torch.empty(n, nh * d, dtype=torch.bfloat16, device=DEV)
    K.paged_attention(qkv, want, kc, vc, bt, cu, starts, b, n, nh, nkv, d, 1 / math.sqrt(d), max(q_lens), kernel="mma")
    got = torch.full_like(want, float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(DEV)[0]
    assert _call(fn, qkv, got, kc, vc, bt, cu, starts, b, n, nh, nkv, d, 0, max(q_lens), 1) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(DEV)[0] == free_before
    assert torch.equal(got, want)


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib, fn = _symbol()
    b, nh, nkv, d, ps, splits = 64, 28, 4, 128, 16, 16  # 64*28*16*130*4 bytes = 14.9 MB > 8 MiB
    qkv, kc, vc, bt, cu, starts = _case(3, torch.bfloat16, b, nh, nkv, d, ps, 64)
    out = torch.zeros(b, nh * d, dtype=torch.bfloat16, device=DEV)
    rc = _call(fn, qkv, out, kc, vc, bt, cu, starts, b, b, nh, nkv, d, 0, 1, splits)
    torch.cuda.synchronize()
    assert rc == 4  # EMS_ERR_SCRATCH: nothing was launched
    assert float(out.abs().max()) == 0.0
