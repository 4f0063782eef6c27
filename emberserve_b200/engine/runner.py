"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step(rows)`` takes any mix of rows: portions of prompts of any length
beside single decoded tokens.  It runs only the tokens it is given, as one packed batch,
against what earlier steps left in the cache, writes their keys and values there, and
returns float32 logits at the wanted places.  It is a pure function of (weights, cache
contents, rows): the scheduler, the replay tool and the tests all call this one function.

The reference's equivalent is ``LLMEngine._plan_inputs`` / ``_materialize`` / ``_forward``
(``emberserve/engine.py:917-1016,752-763``) and ``step_logits`` (``:883-900``): packed
tokens, positions, block tables and logit rows, copied to the device from pinned memory.
Here all of a step's integers travel in ONE int32 buffer, and slot numbers are not sent
at all: the cache-write kernel derives them from the block tables.

Pages are reserved by the caller through ``runner.cache`` (``admit`` / ``extend``) before
the step; the step commits what it computed, which lets windowed groups give pages back.
"""

from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass, field

import numpy as np
import torch

from emberserve_b200 import kernels as K
from emberserve_b200.cache.manager import CacheManager, plan_groups
from emberserve_b200.cache.storage import CacheStorage
from emberserve_b200.config.model import ModelConfig
from emberserve_b200.engine.memory import MemoryPlan, plan_memory
from emberserve_b200.parts.base import PagedKV, StepContext
from emberserve_b200.parts.decoder import Decoder
from emberserve_b200.parts.linear import strict_matmul_precision
from emberserve_b200.registry import build_decoder, load_config
from emberserve_b200.weights.loader import init_random_on_device, load_weights

_MIN_PAGES = 64
# How many tokens of one step may wait on the device for the step after it.
MAX_DEFERRED_TOKENS = 8192


@dataclass
class StepRow:
    seq_id: int
    tokens: list[int]
    start: int  # tokens of the request already in the cache
    want: list[int] = field(default_factory=list)  # places among `tokens` whose logits are wanted


class ScratchArena:
    """Named buffers that live across steps; a request for more than a buffer holds
    replaces it with a larger one.

    With `guard` > 0 every buffer gets that many extra elements before and after it, filled
    with a pattern that `verify()` looks for again: a kernel that writes outside the buffer it
    was given shows up there (a debugging aid; compute-sanitizer's memcheck does the same where
    it can be run)."""

    _PATTERN = 0x5A

    def __init__(self, device: torch.device, guard: int = 0) -> None:
        self.device = device
        self.guard = guard
        self._bufs: dict[tuple[str, torch.dtype], torch.Tensor] = {}
        self._whole: dict[tuple[str, torch.dtype], torch.Tensor] = {}
        # Set while CUDA graphs hold pointers into the buffers: a buffer that has to grow then
        # leaves its old memory alive (in `_retired`) for the graphs that were captured over it.
        self.frozen = False
        self._retired: list[torch.Tensor] = []

    def __call__(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= s
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < numel:
            if self.frozen and buf is not None:
                self._retired.append(self._whole.get(key, buf))
            if self.guard:
                # guards of a multiple of 16 bytes keep the buffer as aligned as the allocation
                g = -(-self.guard * dtype.itemsize // 16) * 16 // dtype.itemsize
                whole = torch.empty(max(numel, 1) + 2 * g, dtype=dtype, device=self.device)
                whole.view(torch.uint8).fill_(self._PATTERN)
                self._whole[key] = whole
                buf = whole[g:g + max(numel, 1)]
            else:
                buf = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:numel].view(shape)

    def verify(self) -> None:
        """Raise if the elements around a buffer no longer hold the pattern (guard > 0)."""
        for (name, dtype), whole in self._whole.items():
            n = self._bufs[(name, dtype)].numel()
            g = (whole.numel() - n) // 2
            raw = whole.view(torch.uint8)
            size = dtype.itemsize
            for what, part in (("before", raw[:g * size]), ("after", raw[(g + n) * size:])):
                if bool((part != self._PATTERN).any()):
                    where = int((part != self._PATTERN).nonzero()[0])
                    raise RuntimeError(f"scratch buffer {name!r} ({dtype}): something wrote {what} it "
                                       f"(byte {where} of the guard)")

    def bytes(self) -> int:
        return (sum(b.numel() * b.element_size() for b in self._bufs.values())
                + sum(b.numel() * b.element_size() for b in self._retired))


def _align4(n: int) -> int:
    return (n + 3) & ~3


class ModelRunner:
    # The product runs on a CUDA GPU only.  Tests of the host-side logic subclass the runner
    # with this switched off and the kernels replaced by their plain references.
    _require_cuda = True

    def __init__(self, config: ModelConfig, decoder: Decoder, dtype: torch.dtype,
                 device: str | torch.device = "cuda:0", page_size: int = 16,
                 num_pages: int | None = None, max_pages: int | None = None,
                 num_state_slots: int = 256, gpu_memory_utilization: float = 0.90,
                 reserve_bytes: int | None = None, max_step_tokens: int = 8192, max_graph_rows: int = 256,
                 max_logit_rows: int = 256, scratch_guard: int = 0,
                 tiled_weight_copies: bool | None = None) -> None:
        self.device = torch.device(device)
        if self._require_cuda and (self.device.type != "cuda" or not torch.cuda.is_available()):
            raise RuntimeError("emberserve_b200 runs on a CUDA GPU only; there is no CPU path "
                               f"(device={device!r}, cuda available={torch.cuda.is_available()})")
        self._on_cuda = self.device.type == "cuda"
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {dtype}")
        if decoder.embed is None:
            raise RuntimeError("the decoder has no weights bound; load or initialise them first")
        strict_matmul_precision()
        self.config = config
        self.decoder = decoder
        self.dtype = dtype
        self.page_size = page_size
        self.vocab_size = decoder.spec.vocab_size
        self.max_positions = decoder.spec.max_positions
        self.tiled_weight_bytes = self._give_tiled_twins(tiled_weight_copies)
        self.groups = plan_groups(decoder.cache_entries())
        paged = [g for g in self.groups if g.paged]
        has_state = any(not g.paged for g in self.groups)
        self.memory_plan: MemoryPlan | None = None
        if num_pages is None:
            num_pages = self._pages_from_free_memory(paged, gpu_memory_utilization, reserve_bytes,
                                                     max_step_tokens, max_graph_rows, max_logit_rows,
                                                     num_state_slots if has_state else 0)
            if max_pages is not None:
                num_pages = max(_MIN_PAGES, min(num_pages, max_pages))
        self.num_pages = num_pages
        self.cache = CacheManager(self.groups, num_pages, page_size,
                                  num_state_slots if has_state else 0)
        # One page (and one state slot) more than the manager hands out: rows that pad a
        # CUDA-graph bucket write there.
        self.scratch_page = num_pages
        self.scratch_slot = num_state_slots if has_state else 0
        self.storage = CacheStorage(self.groups, [num_pages + 1] * len(paged), page_size,
                                    num_state_slots + 1 if has_state else 0, dtype, self.device)
        self.scratch = ScratchArena(self.device, guard=scratch_guard)
        self.attn_kernel = "auto"  # "auto", "mma" or "generic": handed to the mixers with every step
        self._meta_dev = torch.empty(1 << 12, dtype=torch.int32, device=self.device)
        self._meta_host = [torch.empty(1 << 12, dtype=torch.int32, pin_memory=self._on_cuda)
                           for _ in range(2)]
        self._meta_events: list[torch.cuda.Event | None] = [None, None]
        self._meta_turn = 0
        # Tokens sampled on the device, for steps that are launched before the host has read
        # them: a token id -(k + 1) in a row stands for token_feedback[k].
        self.token_feedback = torch.zeros(MAX_DEFERRED_TOKENS, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.last_meta_bytes = 0  # bytes of the last step's host-to-device copy
        self.use_graphs = False
        self.graphs = None
        self._has_state = has_state

    def _give_tiled_twins(self, wanted: bool | None) -> int:
        """A second, tiled copy of the weight matrices that decode steps stream, for the
        weight-streaming kernels (`kernels.tile_weight`: they read whole DRAM pages from it and a
        decode step of the 7B shape gets 3 % shorter); the bytes taken.  It costs the weights'
        size again (the embedding not counted unless it is the head too), so by default
        (`wanted` None) it is made
        only where that is at most a tenth of the device's memory; the cache is sized from
        what is left."""
        if wanted is False or not self._on_cuda or self.dtype != torch.bfloat16:
            return 0
        from emberserve_b200.parts.linear import give_tiled_twin

        weights = [w for w in self.decoder.streamed_weights() if K.tile_weight_shape_ok(w)]
        need = sum(w.numel() * w.element_size() for w in weights)
        if wanted is None and need > torch.cuda.get_device_properties(self.device).total_memory // 10:
            return 0
        with torch.cuda.device(self.device):
            return sum(give_tiled_twin(w) for w in weights)

    def enable_graphs(self, max_ctx_len: int, max_rows: int) -> bool:
        """Replay pure-decode steps of up to `max_rows` rows and contexts up to `max_ctx_len`
        from CUDA graphs (captured per row-count bucket at first use).  A mixer with state of
        its own is captured like any other: the slot of each row and the slots to be zeroed
        travel with the step's integers, so its forward must not read them on the host in a
        step of single tokens."""
        from emberserve_b200.engine.graphs import DecodeGraphs

        if not self._on_cuda:
            return False
        self.graphs = DecodeGraphs(self, min(max_ctx_len, self.max_positions), max_rows)
        self.use_graphs = True
        return True

    # ---- construction ----------------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str | os.PathLike, dtype: torch.dtype,
                 device: str | torch.device = "cuda:0", **kw) -> "ModelRunner":
        if cls._require_cuda and not torch.cuda.is_available():
            raise RuntimeError("emberserve_b200 runs on a CUDA GPU only; there is no CPU path")
        config = load_config(model_dir)
        decoder = build_decoder(config)
        load_weights(decoder, model_dir, device, dtype)
        return cls(config, decoder, dtype, device, **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, dtype: torch.dtype,
                    device: str | torch.device = "cuda:0", **kw) -> "ModelRunner":
        if cls._require_cuda and not torch.cuda.is_available():
            raise RuntimeError("emberserve_b200 runs on a CUDA GPU only; there is no CPU path")
        decoder = build_decoder(config)
        init_random_on_device(decoder, seed, device, dtype)
        return cls(config, decoder, dtype, device, **kw)

    def _bytes_per_page(self, paged) -> int:
        esize = torch.empty((), dtype=self.dtype).element_size()
        total = 0
        for g in paged:
            need: PagedKV = g.need
            total += len(g.entries) * 2 * need.num_kv_heads * self.page_size * need.head_dim * esize
        return total

    def _pages_from_free_memory(self, paged, utilization: float, reserve: int | None, max_step_tokens: int,
                                max_graph_rows: int, max_logit_rows: int, state_slots: int) -> int:
        """``emberserve/engine.py:141-153``: (free * utilization - reserve) // bytes per page, the
        reserve being what the steps will allocate AFTER the cache exists (`plan_memory`)."""
        if not paged:
            return _MIN_PAGES
        if not self._on_cuda:
            return 2048  # the reference's fixed page count off the GPU (emberserve/engine.py:194-207)
        free, _ = torch.cuda.mem_get_info(self.device)
        esize = torch.empty((), dtype=self.dtype).element_size()
        state_bytes = 0
        for g in self.groups:
            if not g.paged:
                per_slot = 4
                for d in g.need.shape:
                    per_slot *= d
                state_bytes += len(g.entries) * (state_slots + 1) * per_slot
        self.memory_plan = plan_memory(
            free_bytes=free, utilization=utilization, bytes_per_page=self._bytes_per_page(paged),
            scratch_bytes_per_token=self.decoder.scratch_bytes_per_token(esize), vocab_size=self.vocab_size,
            max_step_tokens=max_step_tokens, max_logit_rows=max_logit_rows, graph_rows=max_graph_rows,
            state_bytes=state_bytes, reserve_override=reserve)
        return max(_MIN_PAGES, self.memory_plan.num_pages)

    # ---- one step ----------------------------------------------------------------------------
    def _check_rows(self, rows: list[StepRow]) -> None:
        seen: set[int] = set()
        for r in rows:
            if r.seq_id in seen:
                raise ValueError(f"request {r.seq_id} appears twice in one step")
            seen.add(r.seq_id)
            if not r.tokens:
                raise ValueError(f"request {r.seq_id} brings no tokens")
            if not self.cache.has_sequence(r.seq_id):
                raise ValueError(f"request {r.seq_id} has no pages; admit it first")
            if r.start != self.cache.committed(r.seq_id):
                raise ValueError(f"request {r.seq_id}: step starts at {r.start} but the cache "
                                 f"holds {self.cache.committed(r.seq_id)} tokens")
            end = r.start + len(r.tokens)
            if end > self.cache.num_tokens(r.seq_id):
                raise ValueError(f"request {r.seq_id}: {end} tokens but pages for "
                                 f"{self.cache.num_tokens(r.seq_id)}; extend it first")
            if end > self.max_positions:
                raise ValueError(f"request {r.seq_id}: position {end - 1} exceeds "
                                 f"max_position_embeddings={self.max_positions}")
            if min(r.tokens) < -MAX_DEFERRED_TOKENS or max(r.tokens) >= self.vocab_size:
                raise ValueError(f"request {r.seq_id}: token id out of vocabulary "
                                 f"(vocab_size {self.vocab_size})")
            for w in r.want:
                if not 0 <= w < len(r.tokens):
                    raise ValueError(f"request {r.seq_id}: wanted place {w} outside its "
                                     f"{len(r.tokens)} tokens")

    def _pack(self, rows: list[StepRow], fresh: list[int] = ()) -> tuple[
            StepContext, list[torch.Tensor], torch.Tensor | None, torch.Tensor, int, torch.Tensor]:
        b = len(rows)
        q_lens = [len(r.tokens) for r in rows]
        starts = [r.start for r in rows]
        n = sum(q_lens)
        cu = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        tokens = np.concatenate([np.asarray(r.tokens, dtype=np.int32) for r in rows])
        positions = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(starts, q_lens)])
        row_of = np.repeat(np.arange(b, dtype=np.int32), q_lens)
        want = np.asarray([cu[i] + w for i, r in enumerate(rows) for w in r.want], dtype=np.int32)
        num_want = int(want.size)
        npaged = len(self.cache.pools)
        tables = []
        for k in range(npaged):
            per_row = [self.cache.table_array(r.seq_id, k) for r in rows]
            width = max(1, max(t.size for t in per_row))
            arr = np.zeros((b, width), dtype=np.int32)
            for i, t in enumerate(per_row):
                arr[i, :t.size] = t  # pages given back read 0: a valid id that is never read
            tables.append(arr)
        slots = np.asarray([max(0, self.cache.state_slot(r.seq_id)) for r in rows], dtype=np.int32)

        sections = [tokens, positions, row_of, cu, np.asarray(starts, dtype=np.int32), want, slots,
                    np.asarray(list(fresh), dtype=np.int32)]
        sections += [t.reshape(-1) for t in tables]
        offsets, total = [], 0
        for s in sections:
            offsets.append(total)
            total += _align4(int(s.size))
        total = max(total, 4)
        if total > self._meta_dev.numel():
            cap = 1 << (total - 1).bit_length()
            if self.scratch.frozen:
                raise RuntimeError("step metadata would outgrow the buffer that graphs hold")
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_host = [torch.empty(cap, dtype=torch.int32, pin_memory=self._on_cuda)
                               for _ in range(2)]
            self._meta_events = [None, None]
        turn = self._meta_turn
        self._meta_turn ^= 1
        if self._meta_events[turn] is not None:
            self._meta_events[turn].synchronize()  # the copy that last read this buffer is done
        host = self._meta_host[turn]
        hv = host.numpy()
        for off, s in zip(offsets, sections):
            hv[off:off + s.size] = s
        self._meta_dev[:total].copy_(host[:total], non_blocking=True)
        self.last_meta_bytes = 4 * total
        if self._on_cuda:
            self._meta_events[turn] = K.record_event()

        def dev(i: int) -> torch.Tensor:
            return self._meta_dev[offsets[i]:offsets[i] + sections[i].size]

        ctx = StepContext(
            num_tokens=n, num_rows=b, dtype=self.dtype, device=self.device,
            tokens=dev(0), positions=dev(1), row_of_token=dev(2), cu_q=dev(3), starts=dev(4),
            q_lens=q_lens, start_list=starts, max_q_len=max(q_lens),
            max_ctx_len=max(s + q for s, q in zip(starts, q_lens)), scratch=self.scratch,
            deferred=self.token_feedback, extra={"attn_kernel": self.attn_kernel})
        bt = [dev(8 + k).view(b, tables[k].shape[1]) for k in range(npaged)]
        return ctx, bt, dev(6), dev(5), num_want, dev(7)

    def verify_scratch(self) -> None:
        """With guarded scratch buffers (scratch_guard > 0): wait for the device and raise if a
        kernel wrote outside a buffer of a step."""
        if not self.scratch.guard:
            return
        if self._on_cuda:
            torch.cuda.synchronize(self.device)
        self.scratch.verify()
        if self.graphs is not None:
            self.graphs.verify_scratch()

    @torch.inference_mode()
    def step(self, rows: list[StepRow]) -> torch.Tensor:
        """Run one step.  Returns float32 logits ``[wanted, vocab]`` in the order of the
        rows and of each row's `want`; the tensor is scratch memory of the runner and is
        valid until the next step."""
        if not rows:
            return torch.empty(0, self.vocab_size, dtype=torch.float32, device=self.device)
        self._check_rows(rows)
        with (torch.cuda.device(self.device) if self._on_cuda else contextlib.nullcontext()):
            # state slots handed out since the last step are zeroed on the device before any
            # mixer reads them; their numbers travel with the step's other integers
            fresh = self.cache.take_fresh_slots() if self._has_state else []
            if self.use_graphs and self.graphs.usable(rows):
                logits = self.graphs.run(rows, fresh)
                for r in rows:
                    self.cache.commit(r.seq_id, r.start + 1)
                self.steps_run += 1
                return logits
            ctx, block_tables, slots, want_rows, num_want, fresh_dev = self._pack(rows, fresh)
            if fresh:
                self.storage.zero_slots(fresh_dev)
            handles = [None if call.cache is None else
                       self.storage.handle(call.cache, call.write, block_tables, slots)
                       for call in self.decoder.spec.order]
            logits = self.decoder.forward(ctx, handles, want_rows, num_want)
        for r in rows:
            self.cache.commit(r.seq_id, r.start + len(r.tokens))
        self.steps_run += 1
        return logits
