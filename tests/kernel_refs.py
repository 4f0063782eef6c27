"""Plain PyTorch restatements of every kernel of ``emberserve_b200.kernels``: same
arguments, same effects, 32-bit (or 64-bit) arithmetic, loops where loops are clearest.

Two uses: the GPU tests compare each CUDA kernel with its restatement here, and the
host-logic tests (no GPU) swap these in for the kernels so that the step function, the
cache and the replay tool can be exercised on the CPU.  Nothing in the package imports
this file.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def embedding(table, tokens, residual, deferred=None):
    n = residual.shape[0]
    tok = tokens[:n].long()
    if deferred is not None and bool((tok < 0).any()):
        tok = torch.where(tok < 0, deferred.long()[(-(tok + 1)).clamp(min=0)], tok)
    residual.copy_(table[tok].float())


def add_rmsnorm(delta, residual, weight, out, eps, rows=None, num_rows=None):
    if rows is None:
        r = residual if delta is None else residual + delta[:residual.shape[0]].float()
        if delta is not None:
            residual.copy_(r)
    else:
        idx = rows[: (rows.numel() if num_rows is None else num_rows)].long()
        r = residual[idx]
        if delta is not None:
            r = r + delta[idx].float()
    y = (r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps)).to(out.dtype).float()
    out[: r.shape[0]].copy_((y * weight.float()).to(out.dtype))


def silu_mul(gate_up, out):
    i = out.shape[1]
    g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def rope_table(inv_freq, max_pos):
    ang = torch.arange(max_pos, dtype=torch.float32, device=inv_freq.device)[:, None] * inv_freq[None, :]
    return torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()


def _rotate(x, cs, rot):
    """x: [N, heads, D] float; cs: [N, rot/2, 2]."""
    half = rot // 2
    c, s = cs[:, None, :, 0], cs[:, None, :, 1]
    x1, x2 = x[..., :half], x[..., half:rot]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]), dim=-1)


def rope_kv_write(qkv, num_heads, num_kv_heads, head_dim, positions, row_of_token, table, rotary_dim,
                  kcache, vcache, block_tables, page_size, write_kv=True):
    n = qkv.shape[0]
    d = head_dim
    q = qkv[:, : num_heads * d].float().view(n, num_heads, d)
    k = qkv[:, num_heads * d:(num_heads + num_kv_heads) * d].float().view(n, num_kv_heads, d)
    v = qkv[:, (num_heads + num_kv_heads) * d:].view(n, num_kv_heads, d)
    pos = positions[:n].long()
    if rotary_dim > 0:
        cs = table[pos]
        q = _rotate(q, cs, rotary_dim)
        k = _rotate(k, cs, rotary_dim)
    qkv[:, : num_heads * d] = q.reshape(n, -1).to(qkv.dtype)
    if not write_kv:
        return
    rows = row_of_token[:n].long()
    page = block_tables[rows, pos // page_size].long()
    slot = pos % page_size
    kcache[page, :, slot, :] = k.to(kcache.dtype)
    vcache[page, :, slot, :] = v.to(vcache.dtype)


def attention_scratch_bytes(num_tokens, num_heads, head_dim, splits):
    return 0 if splits <= 1 else num_tokens * num_heads * splits * (head_dim + 2) * 4


def paged_attention(q, out, kcache, vcache, block_tables, cu_q, starts, num_rows, num_tokens,
                    num_heads, num_kv_heads, head_dim, scale, max_q_len, window=None, splits=1,
                    scratch=None, generic=False, tcgen05=False, kernel="auto", compute_dtype=torch.float32):
    """Per request: gather its keys and values from the pages, dense masked softmax."""
    page_size = kcache.shape[2]
    groups = num_heads // num_kv_heads
    cu = cu_q.tolist()
    st = starts.tolist()
    for b in range(num_rows):
        q0, q1 = cu[b], cu[b + 1]
        qlen, ctx = q1 - q0, st[b] + (q1 - q0)
        if qlen == 0:
            continue
        lo = 0 if not window else max(0, st[b] - window + 1)
        keys = torch.arange(lo, ctx, device=q.device)
        pages = block_tables[b, keys // page_size].long()
        k = kcache[pages, :, keys % page_size, :].to(compute_dtype)  # [T, Hkv, D]
        v = vcache[pages, :, keys % page_size, :].to(compute_dtype)
        qq = q[q0:q1, : num_heads * head_dim].to(compute_dtype).view(qlen, num_heads, head_dim)
        kf = k.repeat_interleave(groups, dim=1).permute(1, 0, 2)
        vf = v.repeat_interleave(groups, dim=1).permute(1, 0, 2)
        scores = torch.matmul(qq.permute(1, 0, 2), kf.transpose(-1, -2)) * scale  # [H, qlen, T]
        qpos = torch.arange(st[b], ctx, device=q.device)[:, None]
        hidden = keys[None, :] > qpos
        if window:
            hidden = hidden | (keys[None, :] <= qpos - window)
        scores = scores.masked_fill(hidden, float("-inf"))
        o = torch.matmul(torch.softmax(scores, dim=-1), vf).permute(1, 0, 2)
        out[q0:q1] = o.reshape(qlen, num_heads * head_dim).to(out.dtype)


def argmax(logits, out):
    out[: logits.shape[0]].copy_(torch.argmax(logits, dim=-1).to(torch.int32))


@torch.inference_mode()  # the logits of a step are inference tensors
def repetition_penalty(logits, row_ptr, token_ids, penalty):
    ptr = row_ptr.tolist()
    for r in range(logits.shape[0]):
        p = float(penalty[r])
        if p == 1.0:
            continue
        for tok in sorted(set(token_ids[ptr[r]:ptr[r + 1]].tolist())):
            s = float(logits[r, tok])
            logits[r, tok] = s / p if s > 0 else s * p


# ---- sampling: Philox4x32-10 and the draw, restated with numpy ----------------------------

def philox4x32_10(key: tuple[int, int], ctr: tuple[int, int, int, int]) -> tuple[int, int, int, int]:
    m0, m1, w0, w1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    k0, k1 = key
    c0, c1, c2, c3 = ctr
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c3 ^ k1) & mask, p0 & mask
        k0, k1 = (k0 + w0) & mask, (k1 + w1) & mask
    return c0, c1, c2, c3


def uniform_of(seed: int, counter: int) -> float:
    seed &= 0xFFFFFFFFFFFFFFFF
    counter &= 0xFFFFFFFFFFFFFFFF
    x = philox4x32_10((seed & 0xFFFFFFFF, seed >> 32), (counter & 0xFFFFFFFF, counter >> 32, 0, 0))[0]
    return float(np.float32(x >> 8) * np.float32(1.0 / 16777216.0))


def kept_mask(z: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """Which tokens survive top-k then top-p (emberserve/sampling.py:56-73), z = logits / T."""
    v = z.numel()
    keep = torch.ones(v, dtype=torch.bool)
    if 0 < top_k < v:
        keep &= z >= torch.topk(z, top_k).values[-1]
    if top_p < 1.0:
        zz = z.masked_fill(~keep, float("-inf")).double()
        probs = torch.softmax(zz, dim=-1)
        order = torch.argsort(zz, descending=True, stable=True)
        sp = probs[order]
        # mass strictly above a token = mass of all tokens with a larger value
        mass_before = torch.zeros(v, dtype=torch.float64)
        csum = torch.cumsum(sp, 0) - sp
        sv = zz[order]
        first_of_value = torch.ones(v, dtype=torch.bool)
        first_of_value[1:] = sv[1:] != sv[:-1]
        idx_first = torch.cummax(torch.where(first_of_value, torch.arange(v), torch.zeros(v, dtype=torch.long)), 0).values
        mass_before[order] = csum[idx_first]
        keep &= mass_before < top_p
    return keep


def sample(logits, temperature, top_k, top_p, seeds, counters, out):
    """Token per row: argmax where temperature == 0, else inverse-CDF draw with the
    Philox uniform, in index order over the kept tokens (32-bit sums, as the kernel)."""
    for r in range(logits.shape[0]):
        x = logits[r].float().cpu()
        t = float(temperature[r])
        if t == 0.0:
            out[r] = int(torch.argmax(x))
            continue
        z = x / np.float32(t)
        keep = kept_mask(z, int(top_k[r]), float(top_p[r]))
        e = torch.where(keep, torch.exp(z - z.max()), torch.zeros_like(z)).double()
        u = uniform_of(int(seeds[r]), int(counters[r]))
        c = torch.cumsum(e, 0)
        target = u * float(c[-1])
        idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64), right=True))
        kept_idx = torch.nonzero(keep).flatten()
        idx = min(idx, int(kept_idx[-1]))
        out[r] = idx


GEMM_SMALLM_MAX_ROWS = 64


def gemm_smallm(x, weight, bias, out, ksplit=1):
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    out.copy_(y.to(out.dtype))


def gemm_smallm_gated(x, weight, out):
    i = out.shape[1]
    y = x.float() @ weight.float().t()
    g, u = y[:, :i], y[:, i:]
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def check_status(clear=True):
    return None


ALL = ["gemm_smallm", "gemm_smallm_gated", "check_status", "embedding", "add_rmsnorm", "silu_mul", "rope_table", "rope_kv_write",
       "attention_scratch_bytes", "paged_attention", "argmax", "repetition_penalty", "sample"]


def install(monkeypatch) -> None:
    """Replace the CUDA kernels of the package by these restatements (host-logic tests)."""
    import sys

    import emberserve_b200.kernels as K

    me = sys.modules[__name__]
    for name in ALL:
        monkeypatch.setattr(K, name, getattr(me, name))
