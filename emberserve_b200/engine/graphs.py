"""CUDA graphs for pure-decode steps.

A step in which every row brings exactly one token has the same launches whatever the
requests are, once the row count is rounded up to a *bucket*: the whole forward pass of a
bucket is captured once and replayed with new integers (tokens, positions, lengths, block
tables) copied into the static buffer it reads.  That removes the launch cost of some
hundred kernels per step, which is what a decode step at small batch is made of.

Rows that pad a bucket are ordinary rows of a one-token request at position 0 whose block
table points at a scratch page that the cache manager never hands out, so no kernel needs
to know about padding (a mixer with state of its own sees a scratch slot for them).  The
split of keys over blocks is fixed per bucket and layer from the largest context a graph
serves; a block whose share of the keys is empty writes an empty partial result, as in the
eager path.

All buckets share ONE arena of scratch buffers: they never run at the same time, so the
buffers are as large as the largest request any bucket makes of them, not the sum.

(The reference does the same with one graph per batch-size bucket and a scratch block,
``emberserve/attn/cuda_graphs.py``; its buckets are over flash-attn / Triton kernels.)
"""

from __future__ import annotations

import gc
from dataclasses import dataclass

import numpy as np
import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import StepContext


def default_buckets(max_rows: int) -> list[int]:
    sizes = [1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512]
    out = [s for s in sizes if s < max_rows]
    out.append(max_rows)
    return out


@dataclass
class _Graph:
    bucket: int
    graph: torch.cuda.CUDAGraph
    meta_dev: torch.Tensor
    host: list[torch.Tensor]
    events: list
    offsets: dict[str, int]
    logits: torch.Tensor
    launches: int
    # Everything the captured launches point into must outlive the graph: the scratch
    # buffers of the bucket (the arena), the context's views and the cache handles.
    keep: tuple = ()
    turn: int = 0


def _forget_cublas_workspaces() -> None:
    clear = getattr(torch._C, "_cuda_clearCublasWorkspaces", None)
    if clear is not None:
        clear()


class DecodeGraphs:
    def __init__(self, runner, max_ctx_len: int, max_rows: int) -> None:
        from emberserve_b200.engine.runner import ScratchArena

        self.runner = runner
        self.max_ctx_len = max_ctx_len
        self.width = runner.cache.pages_needed(max_ctx_len)
        self.buckets = default_buckets(max_rows)
        self.max_rows = max_rows
        self.arena = ScratchArena(runner.device, guard=runner.scratch.guard)
        self._graphs: dict[int, _Graph] = {}
        self._statics: dict[int, tuple] = {}
        self._pool = None
        self.npaged = len(runner.cache.pools)
        self.has_state = runner._has_state

    def usable(self, rows) -> bool:
        if len(rows) > self.max_rows:
            return False
        cache = self.runner.cache
        for r in rows:
            if len(r.tokens) != 1 or r.start + 1 > self.max_ctx_len or len(r.want) > 1:
                return False
            # a request that reserved more pages than the widest table a graph reads (it was
            # admitted for more tokens than max_ctx_len) takes the eager path
            if any(cache.table_array(r.seq_id, k).size > self.width for k in range(self.npaged)):
                return False
        return True

    def _bucket(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        raise AssertionError

    def _layout(self, bucket: int) -> tuple[dict[str, int], int]:
        offsets, total = {}, 0
        sections = [("tokens", bucket), ("positions", bucket), ("row_of", bucket),
                    ("cu", bucket + 1), ("starts", bucket), ("want", bucket)]
        if self.has_state:  # the state slot of each row, and the slots to zero before the step
            sections += [("slots", bucket), ("fresh", bucket)]
        for name, size in sections:
            offsets[name] = total
            total += (size + 3) & ~3
        for k in range(self.npaged):
            offsets[f"bt{k}"] = total
            total += bucket * self.width
        return offsets, total

    def _static(self, bucket: int) -> tuple:
        """The static buffers of a bucket and the context over them, warmed up: two eager
        passes bring library handles and workspaces to life outside the capture and make the
        shared scratch buffers as large as this bucket needs them."""
        if bucket in self._statics:
            return self._statics[bucket]
        r = self.runner
        dev = r.device
        offsets, total = self._layout(bucket)
        meta = torch.zeros(total, dtype=torch.int32, device=dev)
        host = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        for h in host:  # constant sections, and every row a padding row to begin with
            hv = h.numpy()
            hv[offsets["row_of"]:offsets["row_of"] + bucket] = np.arange(bucket)
            hv[offsets["cu"]:offsets["cu"] + bucket + 1] = np.arange(bucket + 1)
            hv[offsets["want"]:offsets["want"] + bucket] = np.arange(bucket)
            for k in range(self.npaged):
                hv[offsets[f"bt{k}"]:offsets[f"bt{k}"] + bucket * self.width] = r.scratch_page
            if self.has_state:
                hv[offsets["slots"]:offsets["slots"] + bucket] = r.scratch_slot
                hv[offsets["fresh"]:offsets["fresh"] + bucket] = r.scratch_slot
        meta.copy_(host[0])

        def view(name: str, size: int) -> torch.Tensor:
            return meta[offsets[name]:offsets[name] + size]

        ctx = StepContext(
            num_tokens=bucket, num_rows=bucket, dtype=r.dtype, device=dev,
            tokens=view("tokens", bucket), positions=view("positions", bucket),
            row_of_token=view("row_of", bucket), cu_q=view("cu", bucket + 1), starts=view("starts", bucket),
            q_lens=[1] * bucket, start_list=[0] * bucket, max_q_len=1, max_ctx_len=self.max_ctx_len,
            scratch=self.arena, extra={"attn_kernel": r.attn_kernel}, deferred=r.token_feedback)
        bts = [view(f"bt{k}", bucket * self.width).view(bucket, self.width) for k in range(self.npaged)]
        slots = view("slots", bucket) if self.has_state else None
        fresh = view("fresh", bucket) if self.has_state else None
        handles = [None if call.cache is None else r.storage.handle(call.cache, call.write, bts, slots)
                   for call in r.decoder.spec.order]
        want = view("want", bucket)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward(ctx, handles, want, bucket, fresh)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self._statics[bucket] = (offsets, meta, host, ctx, bts, handles, want, fresh)
        return self._statics[bucket]

    def _forward(self, ctx, handles, want, bucket: int, fresh) -> torch.Tensor:
        r = self.runner
        if fresh is not None:
            r.storage.zero_slots(fresh)  # slots handed out since the last step (else the scratch slot)
        return r.decoder.forward(ctx, handles, want, bucket)

    def _capture(self, bucket: int) -> _Graph:
        r = self.runner
        offsets, meta, host, ctx, bts, handles, want, fresh = self._static(bucket)
        self.arena.frozen = True  # from here on a buffer that grows leaves its old memory to the graphs
        graph = torch.cuda.CUDAGraph()
        before = K.launch_count()
        # cuBLAS keeps one workspace per stream for as long as the process lives.  One that was
        # allocated inside an earlier capture lies in that graph's memory pool and dangles once
        # the graph is gone (an engine that was dropped): forget the workspaces, so that this
        # capture allocates its own into its own pool, and again afterwards.
        _forget_cublas_workspaces()
        # No cyclic garbage collection while the stream captures: it could free the graphs of an
        # engine that was dropped earlier, and destroying a graph is not permitted during a capture
        # (the capture would be invalidated).  Collect now, then hold the collector off.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self._pool):
                logits = self._forward(ctx, handles, want, bucket, fresh)
        finally:
            if gc_was_on:
                gc.enable()
        _forget_cublas_workspaces()
        if self._pool is None:
            self._pool = graph.pool()
        return _Graph(bucket, graph, meta, host, [None, None], offsets, logits, K.launch_count() - before,
                      keep=(self.arena, ctx, handles, bts, want, fresh))

    def capture_all(self) -> int:
        """Capture every bucket now (largest first), so that no step of a served request pays for
        a capture; returns how many graphs were captured (``emberserve/engine.py:322-334`` captures
        at boot as well)."""
        todo = [b for b in sorted(self.buckets, reverse=True) if b not in self._graphs]
        for bucket in todo:  # every bucket's warm-up first: the shared buffers reach their final sizes
            self._static(bucket)
        for bucket in todo:
            self._graphs[bucket] = self._capture(bucket)
        return len(todo)

    def verify_scratch(self) -> None:
        self.arena.verify()

    def run(self, rows, fresh: list[int] = ()) -> torch.Tensor:
        r = self.runner
        n = len(rows)
        bucket = self._bucket(n)
        g = self._graphs.get(bucket)
        if g is None:
            g = self._graphs[bucket] = self._capture(bucket)
        turn = g.turn
        g.turn ^= 1
        if g.events[turn] is not None:
            g.events[turn].synchronize()
        hv = g.host[turn].numpy()
        o = g.offsets
        hv[o["tokens"]:o["tokens"] + n] = [row.tokens[0] for row in rows]
        starts = [row.start for row in rows]
        hv[o["positions"]:o["positions"] + n] = starts
        hv[o["starts"]:o["starts"] + n] = starts
        if n < bucket:
            hv[o["tokens"] + n:o["tokens"] + bucket] = 0
            hv[o["positions"] + n:o["positions"] + bucket] = 0
            hv[o["starts"] + n:o["starts"] + bucket] = 0
        w = self.width
        for k in range(self.npaged):
            bt = hv[o[f"bt{k}"]:o[f"bt{k}"] + bucket * w].reshape(bucket, w)
            for i, row in enumerate(rows):
                # pages that a window has passed read 0 here: a valid id that no kernel touches
                t = r.cache.table_array(row.seq_id, k)
                bt[i, :t.size] = t
            if n < bucket:
                bt[n:, 0] = r.scratch_page
        if self.has_state:
            hv[o["slots"]:o["slots"] + n] = [r.cache.state_slot(row.seq_id) for row in rows]
            hv[o["slots"] + n:o["slots"] + bucket] = r.scratch_slot
            fresh = list(fresh)
            if len(fresh) > bucket:  # more than the graph's list holds: the rest at once
                r.storage.zero_slots(fresh[bucket:])
                fresh = fresh[:bucket]
            hv[o["fresh"]:o["fresh"] + len(fresh)] = fresh
            hv[o["fresh"] + len(fresh):o["fresh"] + bucket] = r.scratch_slot
        g.meta_dev.copy_(g.host[turn], non_blocking=True)
        g.events[turn] = K.record_event()
        g.graph.replay()
        K.add_launches(g.launches)
        r.last_meta_bytes = 4 * g.meta_dev.numel()
        if all(len(row.want) == 1 for row in rows):
            return g.logits[:n]
        idx = [i for i, row in enumerate(rows) if row.want]
        if not idx:
            return g.logits[:0]
        return g.logits.index_select(0, torch.tensor(idx, device=r.device))
