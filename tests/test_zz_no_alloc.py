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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_static_scratch_entry_equals_the_allocating_one_twice_in_a_row(dtype):
    from emberserve_b200 import kernels as K

    lib, fn = _symbol()
    b, nh, nkv, d, ps, splits = 6, 28, 4, 128, 16, 8
    assert K.attention_scratch_bytes(b, nh, d, splits) <= lib.ems_static_scratch_capacity()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, max_ctx, window) in enumerate([(1, 900, 0), (2, 300, 70)]):
        qkv, kc, vc, bt, cu, starts = _case(seed, dtype, b, nh, nkv, d, ps, max_ctx)
        want = torch.empty(b, nh * d, dtype=dtype, device=DEV)
        scratch = torch.empty(K.attention_scratch_bytes(b, nh, d, splits) // 4, device=DEV)
        K.paged_attention(qkv, want, kc, vc, bt, cu, starts, b, b, nh, nkv, d, 1 / math.sqrt(d), 1,
                          window=window or None, splits=splits, scratch=scratch)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(qkv.data_ptr(), qkv.stride(0), got.data_ptr(), 0 if dtype == torch.float32 else 1,
                kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.shape[1], ps, cu.data_ptr(),
                starts.data_ptr(), b, b, nh, nkv, d, window, 1 / math.sqrt(d), 1, splits, stream)
        torch.cuda.synchronize()
        assert rc == 0, f"call {call}: status {rc}"
        assert torch.cuda.memory_allocated() == before
        tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(got.float(), want.float(), **tol)


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib, fn = _symbol()
    b, nh, nkv, d, ps, splits = 64, 28, 4, 128, 16, 16  # 64*28*16*130*4 bytes = 14.9 MB > 8 MiB
    qkv, kc, vc, bt, cu, starts = _case(3, torch.bfloat16, b, nh, nkv, d, ps, 64)
    out = torch.zeros(b, nh * d, dtype=torch.bfloat16, device=DEV)
    rc = fn(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), 1, kc.data_ptr(), vc.data_ptr(), bt.data_ptr(),
            bt.shape[1], ps, cu.data_ptr(), starts.data_ptr(), b, b, nh, nkv, d, 0, 1 / math.sqrt(d), 1,
            splits, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 4  # EMS_ERR_SCRATCH: nothing was launched
    assert float(out.abs().max()) == 0.0
