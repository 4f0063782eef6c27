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
the engine (``sampling.py:22-39``), moved by ``EngineConfig.seed * 2**32``: two engines with
the same seed draw the same tokens for the same requests in the same order.
"""

from __future__ import annotations

import itertools

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.engine.request import Request

_UNSEEDED_BASE = 0x5EED_0000
_SEED_KEY = "_sampling_seed"


class Sampler:
    def __init__(self, device: torch.device | str, seed: int = 0) -> None:
        self.device = torch.device(device)
        self._unseeded_base = _UNSEEDED_BASE + (int(seed) << 32)
        self._unseeded = itertools.count()
        # the per-row parameters of a step travel in one pinned buffer and one copy (two buffers
        # in turn, each guarded by the event of the copy that last read it)
        self._host: list[torch.Tensor | None] = [None, None]
        self._events: list["torch.cuda.Event | None"] = [None, None]
        self._dev: torch.Tensor | None = None
        self._turn = 0

    def seed_of(self, request: Request) -> int:
        """The request's own seed, or the next one of the engine's; kept with the request."""
        seed = request.metadata.get(_SEED_KEY)
        if seed is None:
            seed = request.sampling_params.seed
            if seed is None:
                seed = self._unseeded_base + next(self._unseeded)
            request.metadata[_SEED_KEY] = int(seed)
        return request.metadata[_SEED_KEY]

    def _upload(self, sections: list[tuple[torch.dtype, list]]) -> list[torch.Tensor]:
        """Device tensors of the given (dtype, values) lists: one host-to-device copy for all of
        them on a CUDA device (each section starts on an 8-byte boundary)."""
        if self.device.type != "cuda":
            return [torch.tensor(v, dtype=dt, device=self.device) for dt, v in sections]
        sizes = [torch.empty((), dtype=dt).element_size() * len(v) for dt, v in sections]
        offsets, total = [], 0
        for size in sizes:
            offsets.append(total)
            total += (size + 7) & ~7
        turn = self._turn
        self._turn ^= 1
        if self._host[turn] is None or self._host[turn].numel() < total:
            self._host[turn] = torch.empty(max(total, 4096), dtype=torch.uint8, pin_memory=True)
            self._events[turn] = None
        if self._dev is None or self._dev.numel() < total:
            self._dev = torch.empty(max(total, 4096), dtype=torch.uint8, device=self.device)
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        host = self._host[turn]
        for (dt, values), off, size in zip(sections, offsets, sizes):
            if size:
                host[off:off + size].view(dt).copy_(torch.tensor(values, dtype=dt))
        self._dev[:total].copy_(host[:total], non_blocking=True)
        self._events[turn] = K.record_event()
        return [self._dev[off:off + size].view(dt) for (dt, _), off, size in zip(sections, offsets, sizes)]

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
        penalised = any(p.repetition_penalty != 1.0 for p in params)
        if all(p.is_greedy for p in params) and not penalised:
            K.argmax(logits, out)
            return out
        sections: list[tuple[torch.dtype, list]] = []
        if penalised:
            ptr, flat = [0], []
            for q, p in zip(requests, params):
                if p.repetition_penalty != 1.0:
                    flat.extend(sorted(set(q.all_token_ids)))
                ptr.append(len(flat))
            sections += [(torch.int32, ptr), (torch.int32, flat or [0]),
                         (torch.float32, [p.repetition_penalty for p in params])]
        greedy = all(p.is_greedy for p in params)
        if not greedy:
            sections += [(torch.float32, [p.temperature for p in params]),
                         (torch.int32, [p.top_k for p in params]),
                         (torch.float32, [p.top_p for p in params]),
                         (torch.int64, [_signed64(self.seed_of(q)) for q in requests]),
                         (torch.int64, [q.num_output_tokens for q in requests])]
        dev = self._upload(sections)
        if penalised:
            K.repetition_penalty(logits, dev[0], dev[1], dev[2])
            dev = dev[3:]
        if greedy:
            K.argmax(logits, out)
        else:
            K.sample(logits, dev[0], dev[1], dev[2], dev[3], dev[4], out)
        return out

    def sample(self, logits: torch.Tensor, requests: list[Request]) -> list[int]:
        return self.sample_tensor(logits, requests).tolist()


def _signed64(x: int) -> int:
    x &= 0xFFFFFFFFFFFFFFFF
    return x - (1 << 64) if x >= (1 << 63) else x
