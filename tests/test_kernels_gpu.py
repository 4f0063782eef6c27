"""Each CUDA kernel alone against its plain restatement (kernel_refs.py), in 32-bit and in
bfloat16, at sizes other than the engine's test models: widths and vocabularies that are
no power of two, head sizes in steps of 16, odd group counts, several page sizes."""

from __future__ import annotations

import math

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def K():
    from emberserve_b200 import kernels

    return kernels


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def test_extension_is_loaded_from_the_tree():
    import os

    path = K().library_path()
    assert os.path.basename(path) == "libemberserve_b200.so"
    with open(f"/proc/{os.getpid()}/maps") as f:
        assert any("libemberserve_b200.so" in line for line in f)


def test_kernels_refuse_cpu_tensors():
    k = K()
    with pytest.raises(k.KernelError):
        k.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,h,v", [(1, 48, 77), (37, 3584, 1000), (5, 1000, 333)])
def test_embedding(dtype, n, h, v):
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(v, h, device=dev(), generator=g).to(dtype)
    tokens = torch.randint(0, v, (n + 3,), device=dev(), generator=g).to(torch.int32)
    got = torch.full((n, h), 7.0, device=dev())
    want = torch.empty_like(got)
    K().embedding(table, tokens, got)
    ref.embedding(table, tokens, want)
    assert torch.equal(got, want)
    # tokens that stand for entries of a device buffer: -(k + 1) reads deferred[k]
    deferred = torch.randint(0, v, (9,), device=dev(), generator=g).to(torch.int32)
    mixed = tokens.clone()
    mixed[::2] = -(torch.arange(mixed[::2].numel(), device=dev(), dtype=torch.int32) % 9 + 1)
    K().embedding(table, mixed, got, deferred=deferred)
    ref.embedding(table, mixed, want, deferred=deferred)
    assert torch.equal(got, want)
    resolved = torch.where(mixed < 0, deferred[(-(mixed + 1)).clamp(min=0).long()], mixed)
    assert torch.equal(got, table[resolved[:n].long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,h,eps", [(1, 64, 1e-6), (9, 1000, 1e-5), (33, 3584, 1e-6), (4, 5120, 3e-6)])
@pytest.mark.parametrize("wdtype", ["same", "f32"])
def test_add_rmsnorm(dtype, n, h, eps, wdtype):
    g = torch.Generator(device="cuda").manual_seed(1)
    delta = (torch.randn(n, h, device=dev(), generator=g) * 2).to(dtype)
    res0 = torch.randn(n, h, device=dev(), generator=g) * 3
    w = (1 + 0.1 * torch.randn(h, device=dev(), generator=g)).to(dtype if wdtype == "same" else torch.float32)
    for d in (delta, None):
        res_a, res_b = res0.clone(), res0.clone()
        out_a = torch.empty(n, h, dtype=dtype, device=dev())
        out_b = torch.empty_like(out_a)
        K().add_rmsnorm(d, res_a, w, out_a, eps)
        ref.add_rmsnorm(d, res_b, w, out_b, eps)
        assert torch.allclose(res_a, res_b, rtol=0, atol=0 if d is None else 1e-6)
        torch.testing.assert_close(out_a.float(), out_b.float(), **tol(dtype))
    # gathered rows: compact output, residual untouched, a row may be wanted twice
    rows = torch.tensor([n - 1, 0, n - 1, 7][: max(1, min(4, n + 1))], device=dev(), dtype=torch.int32) % n
    rows_buf = torch.cat([rows, torch.full((5,), 10**6, device=dev(), dtype=torch.int32)])
    res_a = res0.clone()
    out_a = torch.empty(rows.numel(), h, dtype=dtype, device=dev())
    out_b = torch.empty_like(out_a)
    K().add_rmsnorm(delta, res_a, w, out_a, eps, rows=rows_buf, num_rows=rows.numel())
    ref.add_rmsnorm(delta, res0.clone(), w, out_b, eps, rows=rows_buf, num_rows=rows.numel())
    assert torch.equal(res_a, res0)
    torch.testing.assert_close(out_a.float(), out_b.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,i", [(1, 16), (7, 4864), (130, 18944), (3, 1001), (5, 12)])
def test_silu_mul(dtype, n, i):
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = (torch.randn(n, 2 * i, device=dev(), generator=g) * 3).to(dtype)
    gu[0, :8] = torch.tensor([-1e4, -200.0, -90.0, -30.0, 30.0, 90.0, 200.0, 1e4], device=dev()).to(dtype)  # gates
    got = torch.empty(n, i, dtype=dtype, device=dev())
    want = torch.empty_like(got)
    K().silu_mul(gu, got)
    ref.silu_mul(gu, want)
    assert torch.isfinite(got.float()).all()
    torch.testing.assert_close(got.float(), want.float(), **(tol(dtype) if dtype == torch.float32
                                                              else dict(rtol=8e-3, atol=1e-6)))  # one rounding


@pytest.mark.parametrize("half,theta,max_pos", [(8, 1e4, 128), (64, 1e6, 4096), (24, 5e4, 777)])
def test_rope_table(half, theta, max_pos):
    from emberserve_b200.parts.rope import inv_frequencies

    inv = inv_frequencies(2 * half, theta).to(dev())
    got = K().rope_table(inv, max_pos)
    want = ref.rope_table(inv, max_pos)
    assert got.shape == (max_pos, half, 2)
    # cos/sin of the same float32 angle: only the last bits of the two libraries differ
    torch.testing.assert_close(got, want, rtol=0, atol=2e-6)
    ang64 = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv.cpu()[None, :]
    torch.testing.assert_close(got[..., 0].cpu().double(), ang64.double().cos(), rtol=0, atol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot,ps", [(4, 2, 16, 16, 4), (7, 1, 48, 48, 16), (28, 4, 128, 128, 16),
                                             (3, 3, 32, 16, 8), (5, 1, 80, 0, 1)])
def test_rope_kv_write(dtype, nh, nkv, d, rot, ps):
    g = torch.Generator(device="cuda").manual_seed(3)
    b, max_pos = 3, 200
    q_lens, starts = [5, 1, 9], [3, 150, 0]
    n = sum(q_lens)
    positions = torch.cat([torch.arange(s, s + q) for s, q in zip(starts, q_lens)]).to(dev(), torch.int32)
    row_of = torch.repeat_interleave(torch.arange(b), torch.tensor(q_lens)).to(dev(), torch.int32)
    width = max_pos // ps + 1
    pages = b * width  # every row has pages of its own
    bt = torch.randperm(pages, device=dev(), generator=g).view(b, width).to(torch.int32)
    table = None
    if rot:
        from emberserve_b200.parts.rope import inv_frequencies

        table = K().rope_table(inv_frequencies(rot, 1e4).to(dev()), max_pos)
    qkv = torch.randn(n, (nh + 2 * nkv) * d, device=dev(), generator=g).to(dtype)
    caches = [torch.full((pages, nkv, ps, d), 9.0, dtype=dtype, device=dev()) for _ in range(4)]
    qa, qb = qkv.clone(), qkv.clone()
    K().rope_kv_write(qa, nh, nkv, d, positions, row_of, table, rot, caches[0], caches[1], bt, ps)
    ref.rope_kv_write(qb, nh, nkv, d, positions, row_of, table, rot, caches[2], caches[3], bt, ps)
    t = tol(dtype)
    torch.testing.assert_close(qa.float(), qb.float(), **t)
    torch.testing.assert_close(caches[0].float(), caches[2].float(), **t)
    assert torch.equal(caches[1], caches[3])  # values are copied, bit for bit
    # without the write only q changes
    qc = qkv.clone()
    K().rope_kv_write(qc, nh, nkv, d, positions, row_of, table, rot, None, None, None, ps, write_kv=False)
    assert torch.equal(qc[:, : nh * d], qa[:, : nh * d])
    assert torch.equal(qc[:, nh * d:], qkv[:, nh * d:])


def _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, splits, seed=4, peaky=False, **how):
    g = torch.Generator(device="cuda").manual_seed(seed)
    b = len(q_lens)
    n = sum(q_lens)
    ctx = [s + q for s, q in zip(starts, q_lens)]
    width = max(-(-c // ps) for c in ctx) + 2
    pages = b * width + 5
    perm = torch.randperm(pages, device=dev(), generator=g)[: b * width].view(b, width).to(torch.int32)
    kc = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
    vc = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
    stride = (nh + 2 * nkv) * d
    qkv = torch.randn(n, stride, device=dev(), generator=g)
    if peaky:
        qkv *= 4.0  # sharp softmax: single far keys carry the result
    qkv = qkv.to(dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=dev(), dtype=torch.int32)
    st = torch.tensor(starts, device=dev(), dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    got = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    want = torch.empty_like(got)
    scratch = None
    if splits > 1:
        scratch = torch.empty(K().attention_scratch_bytes(n, nh, d, splits) // 4, device=dev())
    K().paged_attention(qkv, got, kc, vc, perm, cu, st, b, n, nh, nkv, d, scale, max(q_lens),
                        window=window, splits=splits, scratch=scratch, **how)
    ref.paged_attention(qkv, want, kc, vc, perm, cu, st, b, n, nh, nkv, d, scale, max(q_lens),
                        window=window, compute_dtype=torch.float64)
    return got.float(), want.float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,ps", [(4, 2, 16, 4), (3, 1, 32, 8), (7, 1, 48, 16), (28, 4, 128, 16),
                                         (6, 6, 80, 16), (2, 1, 256, 32), (14, 2, 64, 1)])
def test_paged_attention_mixed_rows(dtype, nh, nkv, d, ps):
    """Prompt portions beside decoded tokens, contexts that end inside and at the edge of a
    page and of a key tile."""
    q_lens = [37, 1, 2, 1, 64, 5]
    starts = [0, 63, 30, 128, 17, 95]
    got, want = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, None, 1)
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 32, 33, 100])
def test_paged_attention_window(dtype, window):
    got, want = _attention_case(dtype, 7, 1, 48, 16, [40, 1, 3, 1], [0, 77, 64, 31], window, 1, peaky=True)
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [2, 3, 16])
@pytest.mark.parametrize("window", [None, 70])
def test_paged_attention_decode_splits(dtype, splits, window):
    """Decode rows with the keys split over several blocks; short contexts leave some
    splits empty."""
    q_lens = [1] * 6
    starts = [0, 1, 31, 32, 700, 255]
    got, want = _attention_case(dtype, 28, 4, 128, 16, q_lens, starts, window, splits, peaky=True)
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("nh,nkv,d,ps", [(28, 4, 128, 16), (14, 2, 64, 16), (16, 1, 128, 16), (8, 8, 64, 8),
                                         (7, 1, 128, 4), (6, 3, 64, 32), (12, 4, 128, 1), (4, 2, 64, 48)])
@pytest.mark.parametrize("splits,window", [(1, None), (5, None), (2, 100), (16, 33), (1, 16)])
def test_decode_tensor_core_kernel(nh, nkv, d, ps, splits, window):
    """The bfloat16 tensor-core decode kernel (head sizes 64 and 128, up to 16 query heads per
    KV head, any page size) against the restatement and against the generic kernel; contexts
    of 1 key, at page and tile edges, and long ones."""
    dtype = torch.bfloat16
    q_lens = [1] * 9
    starts = [0, 1, 15, 16, 17, 63, 64, 1500, 700]
    got, want = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, splits, peaky=True)
    torch.testing.assert_close(got, want, **tol(dtype))
    g = torch.Generator(device="cuda").manual_seed(11)
    # the same inputs through the generic kernel
    b, n = len(q_lens), len(q_lens)
    width = max(-(-(s + 1) // ps) for s in starts) + 1
    pages = b * width
    perm = torch.randperm(pages, device=dev(), generator=g).view(b, width).to(torch.int32)
    kc = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
    vc = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
    qkv = (torch.randn(n, (nh + 2 * nkv) * d, device=dev(), generator=g) * 3).to(dtype)
    cu = torch.arange(b + 1, device=dev(), dtype=torch.int32)
    st = torch.tensor(starts, device=dev(), dtype=torch.int32)
    scratch = torch.empty(max(1, K().attention_scratch_bytes(n, nh, d, splits) // 4), device=dev())
    outs = []
    for generic in (False, True):
        out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
        K().paged_attention(qkv, out, kc, vc, perm, cu, st, b, n, nh, nkv, d, 1 / math.sqrt(d), 1,
                            window=window, splits=splits, scratch=scratch, generic=generic)
        outs.append(out.float())
    torch.testing.assert_close(outs[0], outs[1], **tol(dtype))


@pytest.mark.parametrize("nh,nkv,d,ps", [(28, 4, 128, 16), (14, 2, 64, 16), (20, 1, 128, 16), (3, 3, 64, 8),
                                         (7, 1, 128, 4), (6, 3, 64, 32), (8, 4, 128, 1), (2, 1, 64, 48)])
@pytest.mark.parametrize("window", [None, 1, 40, 64, 65, 200])
def test_prefill_tensor_core_kernel(nh, nkv, d, ps, window):
    """The bfloat16 tensor-core kernel for prompt portions (head sizes 64 and 128, any
    group count and page size): fresh prompts, later portions over cached context, single
    tokens, lengths around the 64-key tile and the 16-row warp tile; against the restatement
    and the generic kernel."""
    dtype = torch.bfloat16
    q_lens = [130, 1, 64, 9, 2, 65, 1, 33]
    starts = [0, 200, 64, 119, 0, 63, 0, 300]
    got, want = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, 1, seed=21, peaky=True)
    torch.testing.assert_close(got, want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,d,ps", [(28, 4, 128, 16), (14, 2, 64, 16), (16, 1, 128, 16), (8, 8, 64, 32),
                                         (7, 1, 128, 48), (6, 3, 64, 32), (8, 4, 128, 16), (2, 1, 64, 48)])
@pytest.mark.parametrize("window", [None, 1, 40, 64, 65, 200])
def test_prefill_tcgen05_kernel(nh, nkv, d, ps, window):
    """The tcgen05 kernel for prompt portions (head sizes 64 and 128, pages of a multiple of 16
    keys), forced at every length: rows that end inside a 128-row tile, tiles that span tokens
    of several heads, contexts around the 64-key tile."""
    dtype = torch.bfloat16
    q_lens = [130, 1, 64, 9, 2, 65, 1, 33]
    starts = [0, 200, 64, 119, 0, 63, 0, 300]
    got, want = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, 1, seed=21, peaky=True,
                                tcgen05=True)
    torch.testing.assert_close(got, want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,d,ps,window", [(28, 4, 128, 16, None), (14, 2, 64, 16, 300), (5, 5, 128, 16, None),
                                                (12, 2, 128, 48, 1000), (3, 1, 64, 2, None)])
def test_prefill_tcgen05_kernel_long(nh, nkv, d, ps, window):
    """Long portions (many key tiles, every stage of the K and V rings used many times): the
    tcgen05 kernel where it takes the page size, against the restatement and the generic kernel;
    the default dispatch must agree whichever kernel it picks."""
    dtype = torch.bfloat16
    q_lens = [700, 1, 391]
    starts = [0, 900, 1234]
    how = dict(tcgen05=True) if ps % 16 == 0 else {}
    got, want = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, 1, seed=22, peaky=True, **how)
    torch.testing.assert_close(got, want, **tol(dtype))
    got2, _ = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, 1, seed=22, peaky=True, generic=True)
    torch.testing.assert_close(got, got2, **tol(dtype))
    got3, _ = _attention_case(dtype, nh, nkv, d, ps, q_lens, starts, window, 1, seed=22, peaky=True)
    torch.testing.assert_close(got3, want, **tol(dtype))


def test_prefill_tcgen05_kernel_refuses_other_pages():
    with pytest.raises(Exception, match="paged_attention"):
        _attention_case(torch.bfloat16, 4, 2, 64, 8, [40], [0], None, 1, tcgen05=True)


@pytest.mark.parametrize("kernel", ["auto", "generic", "mma", "tcgen05"])
@pytest.mark.parametrize("window", [None, 90])
def test_attention_ignores_slots_without_a_key(kernel, window):
    """Cache slots behind the end of a context (and pages nobody owns) hold non-numbers: a
    kernel that let them touch a product, even with a zero weight, would return them."""
    dtype, nh, nkv, d, ps = torch.bfloat16, 8, 2, 128, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    q_lens, starts = [300, 70, 1], [0, 201, 333]
    b, n = len(q_lens), sum(q_lens)
    ctx = [s + q for s, q in zip(starts, q_lens)]
    width = max(-(-c // ps) for c in ctx) + 1
    pages = b * width + 3
    perm = torch.randperm(pages, device=dev(), generator=g)[: b * width].view(b, width).to(torch.int32)
    kc = torch.full((pages, nkv, ps, d), float("nan"), dtype=dtype, device=dev())
    vc = torch.full_like(kc, float("nan"))
    for r in range(b):
        first = max(0, starts[r] - window + 1) if window else 0  # older keys: behind every window
        for pos in range(first, ctx[r]):
            page = int(perm[r, pos // ps])
            kc[page, :, pos % ps] = torch.randn(nkv, d, device=dev(), generator=g).to(dtype)
            vc[page, :, pos % ps] = torch.randn(nkv, d, device=dev(), generator=g).to(dtype)
    qkv = torch.randn(n, (nh + 2 * nkv) * d, device=dev(), generator=g).to(dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=dev(), dtype=torch.int32)
    st = torch.tensor(starts, device=dev(), dtype=torch.int32)
    got = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    want = torch.empty_like(got)
    K().paged_attention(qkv, got, kc, vc, perm, cu, st, b, n, nh, nkv, d, 1 / math.sqrt(d), max(q_lens),
                        window=window, kernel=kernel)
    ref.paged_attention(qkv, want, kc, vc, perm, cu, st, b, n, nh, nkv, d, 1 / math.sqrt(d), max(q_lens),
                        window=window, compute_dtype=torch.float64)
    assert torch.isfinite(want.float()).all()
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


def test_prefill_tensor_core_kernel_equals_generic_kernel():
    dtype, nh, nkv, d, ps = torch.bfloat16, 28, 4, 128, 16
    g = torch.Generator(device="cuda").manual_seed(12)
    q_lens, starts = [257, 3, 1], [31, 500, 77]
    b, n = len(q_lens), sum(q_lens)
    width = max(-(-(s + q) // ps) for s, q in zip(starts, q_lens)) + 1
    perm = torch.randperm(b * width, device=dev(), generator=g).view(b, width).to(torch.int32)
    kc = torch.randn(b * width, nkv, ps, d, device=dev(), generator=g).to(dtype)
    vc = torch.randn(b * width, nkv, ps, d, device=dev(), generator=g).to(dtype)
    qkv = (torch.randn(n, (nh + 2 * nkv) * d, device=dev(), generator=g) * 2).to(dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=dev(), dtype=torch.int32)
    st = torch.tensor(starts, device=dev(), dtype=torch.int32)
    outs = []
    for generic in (False, True):
        out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
        K().paged_attention(qkv, out, kc, vc, perm, cu, st, b, n, nh, nkv, d, 1 / math.sqrt(d), max(q_lens),
                            generic=generic)
        outs.append(out.float())
    torch.testing.assert_close(outs[0], outs[1], **tol(dtype))


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_prefill_far_key_stands_out(kernel):
    """A late query of a long prompt whose score for one far key dominates: at the edges of the
    128-key tiles, of the stages of the K/V rings and of the pages."""
    dtype, nh, nkv, d, ps, t = torch.bfloat16, 4, 2, 128, 16, 1500
    qtok = 1400
    for far in (0, 127, 128, 255, 256, 1279, 1280, 1399, 1400):
        g = torch.Generator(device="cuda").manual_seed(far)
        pages = t // ps + 2
        perm = torch.randperm(pages, device=dev(), generator=g)[None, :].to(torch.int32)
        kc = (torch.randn(pages, nkv, ps, d, device=dev(), generator=g) * 0.1).to(dtype)
        vc = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
        qkv = torch.randn(t, (nh + 2 * nkv) * d, device=dev(), generator=g).to(dtype)
        page, slot = int(perm[0, far // ps]), far % ps
        kc[page, 0, slot] = (qkv[qtok, :d].float() * 50.0).to(dtype)  # head 0 of that token points at `far`
        cu = torch.tensor([0, t], device=dev(), dtype=torch.int32)
        st = torch.zeros(1, device=dev(), dtype=torch.int32)
        got = torch.empty(t, nh * d, device=dev(), dtype=dtype)
        want = torch.empty_like(got)
        K().paged_attention(qkv, got, kc, vc, perm, cu, st, 1, t, nh, nkv, d, 1 / math.sqrt(d), t, kernel=kernel)
        ref.paged_attention(qkv, want, kc, vc, perm, cu, st, 1, t, nh, nkv, d, 1 / math.sqrt(d), t,
                            compute_dtype=torch.float64)
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
        # the row really is that one value vector
        torch.testing.assert_close(got[qtok, :d].float(), vc[page, 0, slot].float(), **tol(dtype))


@pytest.mark.parametrize("nh,nkv,d,ps", [(28, 4, 128, 16), (14, 2, 64, 16), (16, 1, 128, 16), (8, 8, 64, 8),
                                         (7, 1, 128, 4), (6, 3, 64, 32), (12, 4, 128, 1), (4, 2, 64, 48)])
@pytest.mark.parametrize("splits,window", [(1, None), (5, None), (2, 100), (16, 33), (1, 16)])
@pytest.mark.parametrize("rotary", [True, False])
def test_decode_attention_fused_equals_the_three_kernels(nh, nkv, d, ps, splits, window, rotary):
    """Rotation of q and k, the write of the new key and value and the attention in one kernel
    against the same done by the rotary kernel and the attention kernel, and against the
    restatement; then once
    more without the write, reading what the first call wrote."""
    from emberserve_b200.parts.rope import inv_frequencies

    dtype = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(31)
    starts = [0, 1, 15, 16, 700, 255, 31]
    b = len(starts)
    width = max(starts) // ps + 2
    pages = b * width + 3
    bt = torch.randperm(pages, device=dev(), generator=g)[: b * width].view(b, width).to(torch.int32)
    kc0 = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
    vc0 = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
    qkv0 = (torch.randn(b, (nh + 2 * nkv) * d, device=dev(), generator=g) * 2).to(dtype)
    rot = d if rotary else 0
    table = K().rope_table(inv_frequencies(d, 1e4).to(dev()), 1024) if rotary else None
    cu = torch.arange(b + 1, device=dev(), dtype=torch.int32)
    st = torch.tensor(starts, device=dev(), dtype=torch.int32)
    rows = torch.arange(b, device=dev(), dtype=torch.int32)
    scale = 1 / math.sqrt(d)

    def scratch():
        return (torch.empty(K().attention_scratch_bytes(b, nh, d, splits) // 4, device=dev()) if splits > 1 else None)

    for write in (True, False):
        # the three kernels
        qa, ka, va = qkv0.clone(), kc0.clone(), vc0.clone()
        K().rope_kv_write(qa, nh, nkv, d, st, rows, table, rot, ka, va, bt, ps, write_kv=write)
        want = torch.empty(b, nh * d, device=dev(), dtype=dtype)
        K().paged_attention(qa, want, ka, va, bt, cu, st, b, b, nh, nkv, d, scale, 1, window=window, splits=splits,
                            scratch=scratch())
        # the one kernel
        kb, vb = kc0.clone(), vc0.clone()
        got = torch.full((b, nh * d), float("nan"), device=dev(), dtype=dtype)
        K().decode_attention_fused(qkv0, got, kb, vb, bt, cu, st, b, nh, nkv, d, scale, table, rot, write,
                                   window=window, splits=splits, scratch=scratch())
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
        assert torch.equal(kb, ka) and torch.equal(vb, va)  # the same rounding of the rotated key
        # the restatement, from the caches the three kernels left
        plain_out = torch.empty_like(want)
        ref.paged_attention(qa, plain_out, ka, va, bt, cu, st, b, b, nh, nkv, d, scale, 1, window=window,
                            compute_dtype=torch.float64)
        torch.testing.assert_close(got.float(), plain_out.float(), **tol(dtype))
        kc0, vc0 = ka, va  # the second round reads the keys that the first one wrote


def test_paged_attention_far_key_stands_out():
    """One far key among hundreds carries the whole result: its score is made to dominate,
    so a kernel that skipped or misplaced it would be plainly wrong."""
    _far_key_case(torch.float32)
    _far_key_case(torch.bfloat16)  # decode rows in bfloat16 run on the tensor-core kernel


def _far_key_case(dtype):
    nh, nkv, d, ps, ctx = 4, 1, 64, 16, 600
    for far in (0, 15, 16, 511, 512, 598):
        g = torch.Generator(device="cuda").manual_seed(far)
        pages = 64
        perm = torch.randperm(pages, device=dev(), generator=g)[None, :].to(torch.int32)
        kc = (torch.randn(pages, nkv, ps, d, device=dev(), generator=g) * 0.1).to(dtype)
        vc = torch.randn(pages, nkv, ps, d, device=dev(), generator=g).to(dtype)
        q = torch.randn(1, (nh + 2) * d, device=dev(), generator=g).to(dtype)
        page, slot = int(perm[0, far // ps]), far % ps
        kc[page, 0, slot] = (q[0, :d].float() * 50.0).to(dtype)  # head 0 points at key `far`
        cu = torch.tensor([0, 1], device=dev(), dtype=torch.int32)
        st = torch.tensor([ctx - 1], device=dev(), dtype=torch.int32)
        out = torch.empty(1, nh * d, device=dev(), dtype=dtype)
        for splits in (1, 4):
            scratch = torch.empty(max(1, K().attention_scratch_bytes(1, nh, d, splits) // 4), device=dev())
            K().paged_attention(q, out, kc, vc, perm, cu, st, 1, 1, nh, nkv, d, 1.0, 1, splits=splits,
                                scratch=scratch)
            t = 1e-4 if dtype == torch.float32 else 2e-2
            torch.testing.assert_close(out[0, :d].float(), vc[page, 0, slot].float(), rtol=t, atol=t)


@pytest.mark.parametrize("r,v", [(1, 7), (5, 1000), (64, 152064), (3, 151936)])
def test_argmax(r, v):
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(r, v, device=dev(), generator=g)
    logits[0, v // 2] = logits[0, v - 1] = 99.0  # a tie: the first index wins
    got = torch.empty(r, dtype=torch.int32, device=dev())
    K().argmax(logits, got)
    assert got.tolist() == torch.argmax(logits, -1).tolist()
    assert got[0].item() == v // 2


def test_repetition_penalty():
    g = torch.Generator(device="cuda").manual_seed(6)
    r, v = 3, 500
    logits = torch.randn(r, v, device=dev(), generator=g)
    ids = [[1, 5, 5, 499], [], [0, 7, 250]]
    ptr = torch.tensor([0, 4, 4, 7], dtype=torch.int32, device=dev())
    flat = torch.tensor([t for row in ids for t in row], dtype=torch.int32, device=dev())
    pen = torch.tensor([1.3, 2.0, 0.7], device=dev())
    want = logits.clone().cpu()
    ref.repetition_penalty(want, ptr.cpu(), flat.cpu(), pen.cpu())
    # the kernel sees each token once: the host passes the set (emberserve/sampling.py:42-53)
    uniq = [sorted(set(row)) for row in ids]
    ptr_u = torch.tensor([0, 3, 3, 6], dtype=torch.int32, device=dev())
    flat_u = torch.tensor([t for row in uniq for t in row], dtype=torch.int32, device=dev())
    K().repetition_penalty(logits, ptr_u, flat_u, pen)
    torch.testing.assert_close(logits.cpu(), want)


@pytest.mark.parametrize("v", [320, 5000, 8192, 9001, 40003, 152064])
def test_sample_matches_restated_draw(v):
    """Temperature, top-k and top-p rows against the restated draw (same Philox uniform,
    same kept set, inverse CDF in index order)."""
    g = torch.Generator(device="cuda").manual_seed(7)
    rows = [(0.0, -1, 1.0), (0.8, -1, 1.0), (1.0, 5, 1.0), (0.7, -1, 0.9), (1.3, 50, 0.5), (0.5, 1, 1.0),
            (1.0, -1, 0.01)]
    r = len(rows)
    logits = torch.randn(r, v, device=dev(), generator=g) * 3
    temp = torch.tensor([x[0] for x in rows], device=dev())
    tk = torch.tensor([x[1] for x in rows], device=dev(), dtype=torch.int32)
    tp = torch.tensor([x[2] for x in rows], device=dev())
    agree = total = 0
    for counter in range(6):
        seeds = torch.tensor([1234 + i for i in range(r)], dtype=torch.int64, device=dev())
        ctrs = torch.full((r,), counter, dtype=torch.int64, device=dev())
        got = torch.empty(r, dtype=torch.int32, device=dev())
        K().sample(logits, temp, tk, tp, seeds, ctrs, got)
        want = torch.empty(r, dtype=torch.int32)
        ref.sample(logits.cpu(), temp.cpu(), tk.cpu(), tp.cpu(), seeds.cpu(), ctrs.cpu(), want)
        keep_ok = True
        for i, (t, k, p) in enumerate(rows):
            if t > 0:
                keep = ref.kept_mask(logits[i].cpu() / t, k, p)
                keep_ok &= bool(keep[got[i].item()])
        assert keep_ok, "a token outside the kept set was drawn"
        agree += sum(int(a == b) for a, b in zip(got.tolist(), want.tolist()))
        total += r
        assert got[0].item() == int(torch.argmax(logits[0]))
        assert got[5].item() == int(torch.argmax(logits[5]))  # top_k = 1
    # 32-bit against 64-bit cumulative sums may disagree on a boundary now and then
    assert agree >= total - 2


def test_sample_distribution_and_seeds():
    """Draws follow softmax(logits / T); the same (seed, counter) gives the same token."""
    v, n = 11, 4000
    logits = torch.tensor([[0.5, 1.0, -1.0, 2.0, 0.0, 0.3, -2.0, 1.5, 0.7, -0.5, 1.1]], device=dev())
    logits = logits.repeat(n, 1)
    temp = torch.full((n,), 0.9, device=dev())
    tk = torch.full((n,), -1, dtype=torch.int32, device=dev())
    tp = torch.ones(n, device=dev())
    seeds = torch.arange(n, dtype=torch.int64, device=dev())
    ctrs = torch.zeros(n, dtype=torch.int64, device=dev())
    out = torch.empty(n, dtype=torch.int32, device=dev())
    K().sample(logits, temp, tk, tp, seeds, ctrs, out)
    again = torch.empty_like(out)
    K().sample(logits, temp, tk, tp, seeds, ctrs, again)
    assert torch.equal(out, again)
    freq = torch.bincount(out.long().cpu(), minlength=v).double() / n
    probs = torch.softmax(logits[0].double().cpu() / 0.9, -1)
    assert float((freq - probs).abs().max()) < 0.03
    for i in (0, 17, 999):
        u = ref.uniform_of(i, 0)
        want = int(torch.searchsorted(torch.cumsum(probs, 0), torch.tensor(u, dtype=torch.float64), right=True))
        assert abs(out[i].item() - want) <= 0 or abs(float(torch.cumsum(probs, 0)[min(want, v - 1)]) - u) < 1e-5


@pytest.mark.parametrize("m,n,k,ksplit", [(1, 256, 128, 1), (8, 4608, 3584, 4), (8, 3584, 3584, 5), (16, 1000, 3584, 1),
                                          (17, 384, 18944, 5), (33, 640, 1024, 2), (64, 3584, 18944, 5), (5, 130, 72, 1),
                                          (8, 37888, 3584, 1), (3, 152064, 896, 1), (64, 256, 64, 1), (2, 128, 4096, 8), (9, 200, 640, 7)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_smallm_tcgen05(m, n, k, ksplit, with_bias):
    """The weight-streaming tcgen05 GEMM for few rows against a float32 product of the same
    bfloat16 inputs: row counts around the MMA's column tiles (16, 32, 64), output widths that
    are no multiple of 128, K that is no multiple of 64, K split over blocks."""
    g = torch.Generator(device="cuda").manual_seed(m * 1000 + n)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(n, device=dev(), generator=g).to(torch.bfloat16) if with_bias else None
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev())
    K().gemm_smallm(x, w, bias, out, ksplit=ksplit)
    torch.cuda.synchronize()
    K().check_status()
    want = x.float() @ w.float().t()
    if with_bias:
        want = want + bias.float()
    scale = float(want.abs().max())
    assert float((out.float() - want).abs().max()) <= 8e-3 * scale + 1e-3, (m, n, k, ksplit)


@pytest.mark.parametrize("m,n,k", [(1, 152064, 896), (8, 1000, 3584), (16, 2048, 1024), (5, 130, 72)])
def test_gemm_smallm_float32_output(m, n, k):
    """The same kernel storing its float32 sums unrounded (the logits of the head), from the
    row-major weight and from its tiled copy: against a float64 product of the same bfloat16 inputs,
    to float32 accuracy."""
    g = torch.Generator(device="cuda").manual_seed(m + n)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    outs = []
    for twin in (None, K().tile_weight(w)):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev())
        K().gemm_smallm(x, w, None, out, ksplit=1, twin=twin)
        torch.cuda.synchronize()
        K().check_status()
        assert float((out.double() - want).abs().max()) <= 2e-5 * float(want.abs().max()) + 1e-6
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    with pytest.raises(AssertionError):  # a split K would have to round or to add in another block
        K().gemm_smallm(x, w, None, outs[0], ksplit=2)


@pytest.mark.parametrize("m,n,k,ksplit", [(1, 256, 512, 2), (8, 4608, 3584, 8), (8, 3584, 3584, 5), (16, 1000, 3584, 7),
                                          (17, 384, 18944, 3), (32, 3584, 18944, 5), (5, 130, 200, 2), (64, 256, 1024, 6)])
def test_gemm_smallm_cluster_split(m, n, k, ksplit):
    """K split over the blocks of a thread-block cluster that push their accumulators into the
    shared memory of the blocks that own the rows (no scratch, one launch); the same bits at
    every call."""
    g = torch.Generator(device="cuda").manual_seed(m * 77 + n)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(n, device=dev(), generator=g).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev())
    before = K().launch_count()
    K().gemm_smallm(x, w, bias, out, ksplit=ksplit)
    assert K().launch_count() - before == 1
    torch.cuda.synchronize()
    K().check_status()
    want = x.float() @ w.float().t() + bias.float()
    assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3
    again = torch.empty_like(out)
    K().gemm_smallm(x, w, bias, again, ksplit=ksplit)
    assert torch.equal(out, again)  # fixed order of additions


@pytest.mark.parametrize("m,n,k,ksplit", [(17, 256, 128, 1), (32, 384, 512, 2), (33, 4608, 3584, 4), (64, 3584, 3584, 5),
                                          (65, 3584, 18944, 4), (128, 3584, 18944, 5), (100, 896, 4864, 8),
                                          (127, 1152, 896, 7), (50, 200, 72, 1), (50, 200, 520, 3), (77, 130, 1000, 6),
                                          (128, 1000, 2048, 8), (20, 128, 256, 8), (5, 300, 640, 2), (96, 5120, 1024, 3)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_midm_tcgen05(m, n, k, ksplit, with_bias):
    """The tcgen05 GEMM for 17..128 rows (one block per SM, partial sums carried into their owners'
    shared memory by bulk copies) against a float32 product of the same bfloat16 inputs: row counts
    around its column tiles (32, 64, 128) and no multiple of four, widths that are no multiple of
    128, K that is no multiple of 64, every cluster size; the same bits at every call."""
    g = torch.Generator(device="cuda").manual_seed(m * 1000 + n)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(n, device=dev(), generator=g).to(torch.bfloat16) if with_bias else None
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev())
    before = K().launch_count()
    K().gemm_midm(x, w, bias, out, ksplit=ksplit)
    assert K().launch_count() - before == 1
    torch.cuda.synchronize()
    K().check_status()
    want = x.float() @ w.float().t()
    if with_bias:
        want = want + bias.float()
    scale = float(want.abs().max())
    assert float((out.float() - want).abs().max()) <= 8e-3 * scale + 1e-3, (m, n, k, ksplit)
    again = torch.empty_like(out)
    K().gemm_midm(x, w, bias, again, ksplit=ksplit)
    assert torch.equal(out, again)  # fixed order of additions


def test_tiled_weight_copy_changes_no_bit():
    """The tiled copy of a weight (`kernels.tile_weight`: tile (r, kt) of 128 x 64 contiguous at index
    r * K/64 + kt) holds the same numbers, and the three weight-streaming kernels produce the same
    bits from it as from the row-major matrix; shapes without a tiled form have none."""
    g = torch.Generator(device="cuda").manual_seed(3)
    n, k = 384, 448
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    twin = K().tile_weight(w)
    assert twin.shape == (n * (k // 64), 64)
    for r, kt in [(0, 0), (1, 3), (2, 6)]:
        tile = twin[(r * (k // 64) + kt) * 128:][:128]
        assert torch.equal(tile, w[r * 128:(r + 1) * 128, kt * 64:(kt + 1) * 64])
    assert K().tile_weight(w[:, :400].contiguous()) is None and K().tile_weight(w[:200].contiguous()) is None
    assert K().tile_weight(w.float()) is None
    for m, n, k, ksplit in [(8, 3584, 3584, 8), (3, 256, 128, 1), (16, 4608, 3584, 7), (13, 1152, 896, 3)]:
        x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
        bias = torch.randn(n, device=dev(), generator=g).to(torch.bfloat16)
        twin = K().tile_weight(w)
        a, b = torch.empty(m, n, dtype=torch.bfloat16, device=dev()), torch.empty(m, n, dtype=torch.bfloat16, device=dev())
        K().gemm_smallm(x, w, bias, a, ksplit=ksplit)
        K().gemm_smallm(x, w, bias, b, ksplit=ksplit, twin=twin)
        assert torch.equal(a, b), ("smallm", m, n, k)
    for m, n, k, ksplit in [(17, 3584, 18944, 4), (64, 896, 4864, 8), (96, 256, 128, 1), (128, 1152, 896, 5)]:
        x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
        twin = K().tile_weight(w)
        a, b = torch.empty(m, n, dtype=torch.bfloat16, device=dev()), torch.empty(m, n, dtype=torch.bfloat16, device=dev())
        K().gemm_midm(x, w, None, a, ksplit=ksplit)
        K().gemm_midm(x, w, None, b, ksplit=ksplit, twin=twin)
        assert torch.equal(a, b), ("midm", m, n, k)
    for m, inter, k in [(8, 18944, 3584), (1, 4864, 896), (40, 256, 128), (64, 1280, 512)]:
        x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
        w = (torch.randn(2 * inter, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
        twin = K().tile_weight(w)
        a, b = torch.empty(m, inter, dtype=torch.bfloat16, device=dev()), torch.empty(m, inter, dtype=torch.bfloat16, device=dev())
        K().gemm_smallm_gated(x, w, a)
        K().gemm_smallm_gated(x, w, b, twin=twin)
        assert torch.equal(a, b), ("gated", m, inter, k)
    for m, inter, k in [(100, 1280, 512), (256, 4864, 896), (300, 256, 128)]:
        x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
        w = (torch.randn(2 * inter, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
        twin = K().tile_weight(w)
        a, b = torch.empty(m, inter, dtype=torch.bfloat16, device=dev()), torch.empty(m, inter, dtype=torch.bfloat16, device=dev())
        K().gemm_large_gated(x, w, a)
        K().gemm_large_gated(x, w, b, twin=twin)
        assert torch.equal(a, b), ("two-SM gated", m, inter, k)
    torch.cuda.synchronize()
    K().check_status()


def test_gemm_midm_split_fits_the_device():
    """The K split that `linear` picks for the kernel above lets all clusters of the product start
    at once, and the products it hands to the kernel equal the library's."""
    from emberserve_b200.parts import linear as L

    for m, n, k in [(17, 3584, 18944), (64, 896, 4864), (96, 5120, 27648), (40, 1536, 8960)]:
        split = L.midm_ksplit(m, n, k)
        assert 1 <= split <= 8 and -(-n // 128) <= K().gemm_midm_max_clusters(m, split)
        g = torch.Generator(device="cuda").manual_seed(n)
        x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev(), generator=g) * 0.02).to(torch.bfloat16)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev())
        assert L._use_midm(x, w, None, out) == split
        before = K().launch_count()
        L.linear(x, w, None, out, scratch=lambda *a: None)
        assert K().launch_count() - before == 1  # the kernel of this library, not cuBLAS
        want = x.float() @ w.float().t()
        assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3
    # squarer products and more rows stay with the library
    x = torch.zeros(64, 3584, dtype=torch.bfloat16, device=dev())
    assert L._use_midm(x, torch.zeros(4608, 3584, dtype=torch.bfloat16, device=dev()), None,
                       torch.empty(64, 4608, dtype=torch.bfloat16, device=dev())) == 0
    x = torch.zeros(128, 4864, dtype=torch.bfloat16, device=dev())
    assert L._use_midm(x, torch.zeros(896, 4864, dtype=torch.bfloat16, device=dev()), None,
                       torch.empty(128, 896, dtype=torch.bfloat16, device=dev())) == 0


@pytest.mark.parametrize("m,n,k,ksplit", [(8, 3584, 3584, 5), (1, 896, 4864, 8), (16, 3584, 18944, 5), (5, 200, 640, 1),
                                          (8, 5120, 1024, 2), (13, 130, 512, 3)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_smallm_begins_the_norm_behind_it(m, n, k, ksplit, with_bias):
    """The product added into the float32 residual stream in the kernel's epilogue, with the gain
    of the norm behind it applied to a bfloat16 copy and the rows' sums of squares left in
    per-block shares: against the same done in float64."""
    g = torch.Generator(device="cuda").manual_seed(m * 13 + n)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(n, device=dev(), generator=g).to(torch.bfloat16) if with_bias else None
    gain = (1 + 0.3 * torch.randn(n, device=dev(), generator=g)).to(torch.bfloat16)
    res0 = torch.randn(m, n, device=dev(), generator=g) * 2
    res = res0.clone()
    parts = -(-n // 128) * ksplit
    scaled = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev())
    sumsq = torch.full((parts, 16), float("nan"), device=dev())
    K().gemm_smallm(x, w, bias, None, ksplit=ksplit, norm_behind=K().NormBehind(res, gain, scaled, sumsq))
    torch.cuda.synchronize()
    K().check_status()
    y = x.double() @ w.double().t() + (bias.double() if with_bias else 0)
    want = res0.double() + y
    tol_y = 8e-3 * float(y.abs().max()) + 1e-3  # (the product itself is bfloat16 x bfloat16 in float32)
    assert float((res.double() - want).abs().max()) <= tol_y
    torch.testing.assert_close(scaled.float(), (res * gain.float()).to(torch.bfloat16).float(), rtol=8e-3, atol=1e-6)
    got_sq = sumsq[:, :m].double().sum(0)
    torch.testing.assert_close(got_sq, res.double().pow(2).sum(1), rtol=1e-5, atol=1e-5)
    again_res, again_sq = res0.clone(), torch.empty_like(sumsq)
    K().gemm_smallm(x, w, bias, None, ksplit=ksplit, norm_behind=K().NormBehind(again_res, gain, torch.empty_like(scaled), again_sq))
    assert torch.equal(again_res, res) and torch.equal(again_sq[:, :m], sumsq[:, :m])  # fixed order of additions


@pytest.mark.parametrize("m,n,k,ksplit,parts", [(8, 4608, 3584, 4, 140), (1, 1152, 896, 1, 7), (16, 640, 1024, 2, 33),
                                                (5, 130, 512, 3, 1)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_smallm_finishes_the_norm_before_it(m, n, k, ksplit, parts, gated):
    """Rows of the product multiplied by rsqrt(mean square + eps), the mean square coming from
    per-block shares, before the bias (plain product) or before SiLU (gated product): against
    the norm applied to the activations first, in float64."""
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n + parts)
    r = torch.randn(m, k, device=dev(), generator=g) * 3  # the residual rows that the norm is about
    gain = (1 + 0.3 * torch.randn(k, device=dev(), generator=g)).to(torch.bfloat16)
    xg = (r * gain.float()).to(torch.bfloat16)
    # their sums of squares, cut into `parts` shares (and rubbish in the rows beyond m)
    cut = torch.rand(parts, m, device=dev(), generator=g) + 0.1
    shares = torch.full((parts, 16), float("nan"), device=dev())
    shares[:, :m] = cut / cut.sum(0) * r.pow(2).sum(1)
    eps = 1e-5
    before = K().NormBefore(shares, parts, k, eps)
    rstd = torch.rsqrt(r.double().pow(2).mean(1) + eps)
    if gated:
        inter = n // 2
        w = (torch.randn(2 * inter, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
        out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=dev())
        K().gemm_smallm_gated(xg, w, out, norm_before=before)
        y = (xg.double() * rstd[:, None]) @ w.double().t()
        want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    else:
        w = (torch.randn(n, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
        bias = torch.randn(n, device=dev(), generator=g).to(torch.bfloat16)
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev())
        K().gemm_smallm(xg, w, bias, out, ksplit=ksplit, norm_before=before)
        want = (xg.double() * rstd[:, None]) @ w.double().t() + bias.double()
    torch.cuda.synchronize()
    K().check_status()
    assert float((out.double() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3


@pytest.mark.parametrize("m,inter,k", [(300, 256, 128), (2048, 1152, 896), (513, 4864, 896), (65, 128, 72),
                                       (1000, 2560, 3584), (256, 128, 64), (129, 384, 200)])
def test_gemm_large_gated(m, inter, k):
    """The two-SM kernel of prompt steps (256 x 256 tiles over a pair of blocks, two accumulators
    in tensor memory, silu(gate) * up in the epilogue), against the float32 computation of the
    same bfloat16 inputs: rows that end inside a tile and inside the peer's half, K that ends
    inside a stage, more tiles than SM pairs (both accumulators and every stage used again)."""
    g = torch.Generator(device="cuda").manual_seed(m * 31 + inter)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    out = torch.full((m + 3, inter), float("nan"), dtype=torch.bfloat16, device=dev())
    assert K().gemm_large_gated_supported(m, inter, k)
    K().gemm_large_gated(x, w, out[:m])
    torch.cuda.synchronize()
    K().check_status()
    y = x.float() @ w.float().t()
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    assert float((out[:m].float() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3
    assert bool(torch.isnan(out[m:].float()).all())  # nothing is written past the last row
    again = torch.empty_like(out[:m])
    K().gemm_large_gated(x, w, again)
    assert torch.equal(out[:m], again)


def test_gemm_large_gated_one_row_stands_out():
    """Each output comes from its own token row and its own weight rows: one (token, feature)
    pair is made large and must land at exactly that place."""
    m, inter, k = 700, 640, 256
    x = torch.zeros(m, k, dtype=torch.bfloat16, device=dev())
    w = torch.zeros(2 * inter, k, dtype=torch.bfloat16, device=dev())
    for tok, feat in ((0, 0), (127, 127), (128, 128), (255, 639), (256, 1), (699, 300), (511, 512)):
        x[tok, tok % k] = 2.0
        w[feat, tok % k] += 3.0          # gate = 6
        w[inter + feat, tok % k] += 0.5  # up = 1
    out = torch.empty(m, inter, dtype=torch.bfloat16, device=dev())
    K().gemm_large_gated(x, w, out)
    torch.cuda.synchronize()
    K().check_status()
    y = x.float() @ w.float().t()
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    assert int((want != 0).sum()) >= 7
    assert torch.allclose(out.float(), want, rtol=1e-2, atol=1e-6)


def test_gemm_large_gated_refuses():
    assert not K().gemm_large_gated_supported(512, 200, 128)   # I not a multiple of 128
    assert not K().gemm_large_gated_supported(512, 256, 100)   # K not a multiple of 8
    x = torch.zeros(512, 128, dtype=torch.bfloat16, device=dev())
    w = torch.zeros(400, 128, dtype=torch.bfloat16, device=dev())
    with pytest.raises(Exception):
        K().gemm_large_gated(x, w, torch.empty(512, 200, dtype=torch.bfloat16, device=dev()))


@pytest.mark.parametrize("m,inter,k", [(1, 256, 128), (8, 18944, 3584), (16, 1000, 3584), (17, 4864, 896),
                                       (33, 640, 1024), (64, 2048, 512), (5, 130, 72)])
def test_gemm_smallm_gated(m, inter, k):
    """Gate and up projections and silu(gate) * up in one kernel (two accumulators in tensor
    memory), against the float32 computation of the same bfloat16 inputs."""
    g = torch.Generator(device="cuda").manual_seed(m * 31 + inter)
    x = torch.randn(m, k, device=dev(), generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=dev(), generator=g) * 0.05).to(torch.bfloat16)
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=dev())
    K().gemm_smallm_gated(x, w, out)
    torch.cuda.synchronize()
    K().check_status()
    y = x.float() @ w.float().t()
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3
