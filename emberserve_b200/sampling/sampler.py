"""Turns float32 logits ``[rows, vocab]`` into one token per row, on the device.

Greedy rows take the first maximum; the others are divided by the temperature, filtered
by top-k and top-p, and drawn (``emberserve/sampling.py:110-145``); a repetition penalty,
where asked for, is applied first over the set of the request's tokens (``:42-53``).  All
of it runs in the kernels of ``csrc/sampling.cu``; one device-to-host copy per step
brings the tokens back (``sampling.py:108``).

The draw is counter-based: row i uses the uniform number Philox(seed_i, n_i) where n_i is
how many tokens the request has produced so far.  Its tokens therefore depend on its seed
and its logits only: not on the batch, not on how its prompt was cut, and they survive a
preemption.  Requests without a seed get ``0x5EED0000 + k`` for the k-th such request of
the process (``sampling.py:22-39``).
"""

from __future__ import annotations

import itertools

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.engine.request import Request

_UNSEEDED_BASE = 0x5EED_0000
_unseeded = itertools.count()
_SEED_KEY = "_sampling_seed"


def seed_of(request: Request) -> int:
    seed = request.metadata.get(_SEED_KEY)
    if seed is None:
        seed = request.sampling_params.seed
        if seed is None:
            seed = _UNSEEDED_BASE + next(_unseeded)
        request.metadata[_SEED_KEY] = int(seed)
    return request.metadata[_SEED_KEY]


class Sampler:
    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)

    def sample_tensor(self, logits: torch.Tensor, requests: list[Request],
                      out: torch.Tensor | None = None) -> torch.Tensor:
        """int32 tokens ``[rows]`` on the device (in `out` if given); `logits` may be modified
        in place."""
        r = logits.shape[0]
        assert logits.dim() == 2 and r == len(requests), (tuple(logits.shape), len(requests))
        params = [q.sampling_params for q in requests]
        if out is None:
            out = torch.empty(r, dtype=torch.int32, device=self.device)
        assert out.dtype == torch.int32 and out.numel() == r and out.is_contiguous()
        if any(p.repetition_penalty != 1.0 for p in params):
            ptr, flat = [0], []
            for q, p in zip(requests, params):
                if p.repetition_penalty != 1.0:
                    flat.extend(sorted(set(q.all_token_ids)))
                ptr.append(len(flat))
            K.repetition_penalty(
                logits, torch.tensor(ptr, dtype=torch.int32, device=self.device),
                torch.tensor(flat or [0], dtype=torch.int32, device=self.device),
                torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32,
                             device=self.device))
        if all(p.is_greedy for p in params):
            K.argmax(logits, out)
            return out
        K.sample(
            logits,
            torch.tensor([p.temperature for p in params], dtype=torch.float32, device=self.device),
            torch.tensor([p.top_k for p in params], dtype=torch.int32, device=self.device),
            torch.tensor([p.top_p for p in params], dtype=torch.float32, device=self.device),
            torch.tensor([_signed64(seed_of(q)) for q in requests], dtype=torch.int64, device=self.device),
            torch.tensor([q.num_output_tokens for q in requests], dtype=torch.int64, device=self.device),
            out)
        return out

    def sample(self, logits: torch.Tensor, requests: list[Request]) -> list[int]:
        return self.sample_tensor(logits, requests).tolist()


def _signed64(x: int) -> int:
    x &= 0xFFFFFFFFFFFFFFFF
    return x - (1 << 64) if x >= (1 << 63) else x
