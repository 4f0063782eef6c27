"""CUDA graphs for pure-decode steps.

A step in which every row brings exactly one token has the same launches whatever the
requests are, once the row count is rounded up to a *bucket*: the whole forward pass of a
bucket is captured once and replayed with new integers (tokens, positions, lengths, block
tables) copied into the static buffer it reads.  That removes the launch cost of some
hundred kernels per step, which is what a decode step at small batch is made of.

Rows that pad a bucket are ordinary rows of a one-token request at position 0 whose block
table points at a scratch page that the cache manager never hands out, so no kernel needs
to know about padding.  The split of keys over blocks is fixed per bucket from the
largest context a graph serves; a block whose share of the keys is empty writes an empty
partial result, as in the eager path.

(The reference does the same with one graph per batch-size bucket and a scratch block,
``emberserve/attn/cuda_graphs.py``; its buckets are over flash-attn / Triton kernels.)
"""

from __future__ import annotations

import gc
from dataclasses import dataclass

import numpy as np
import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.attention import decode_splits
from emberserve_b200.parts.base import PagedKV, StepContext


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
        self._arena_cls = ScratchArena
        self._graphs: dict[int, _Graph] = {}
        self._pool = None
        self.npaged = len(runner.cache.pools)

    def usable(self, rows) -> bool:
        if len(rows) > self.max_rows:
            return False
        for r in rows:
            if len(r.tokens) != 1 or r.start + 1 > self.max_ctx_len or len(r.want) > 1:
                return False
        return True

    def _bucket(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        raise AssertionError

    def _layout(self, bucket: int) -> tuple[dict[str, int], int]:
        offsets, total = {}, 0
        for name, size in (("tokens", bucket), ("positions", bucket), ("row_of", bucket),
                           ("cu", bucket + 1), ("starts", bucket), ("want", bucket)):
            offsets[name] = total
            total += (size + 3) & ~3
        for k in range(self.npaged):
            offsets[f"bt{k}"] = total
            total += bucket * self.width
        return offsets, total

    def _capture(self, bucket: int) -> _Graph:
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
        meta.copy_(host[0])

        def view(name: str, size: int) -> torch.Tensor:
            return meta[offsets[name]:offsets[name] + size]

        kv_heads = max((g.need.num_kv_heads for g in r.groups if isinstance(g.need, PagedKV)), default=1)
        arena = self._arena_cls(dev, guard=r.scratch.guard)
        ctx = StepContext(
            num_tokens=bucket, num_rows=bucket, dtype=r.dtype, device=dev,
            tokens=view("tokens", bucket), positions=view("positions", bucket),
            row_of_token=view("row_of", bucket), cu_q=view("cu", bucket + 1), starts=view("starts", bucket),
            q_lens=[1] * bucket, start_list=[0] * bucket, max_q_len=1, max_ctx_len=self.max_ctx_len,
            scratch=arena, extra={"decode_splits": decode_splits(bucket, kv_heads, self.max_ctx_len),
                                    "attn_kernel": r.attn_kernel},
            deferred=r.token_feedback)
        bts = [view(f"bt{k}", bucket * self.width).view(bucket, self.width) for k in range(self.npaged)]
        handles = [None if call.cache is None else r.storage.handle(call.cache, call.write, bts, None)
                   for call in r.decoder.spec.order]
        want = view("want", bucket)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):  # library handles and workspaces come to life outside the capture
            for _ in range(2):
                r.decoder.forward(ctx, handles, want, bucket)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
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
                logits = r.decoder.forward(ctx, handles, want, bucket)
        finally:
            if gc_was_on:
                gc.enable()
        _forget_cublas_workspaces()
        if self._pool is None:
            self._pool = graph.pool()
        return _Graph(bucket, graph, meta, host, [None, None], offsets, logits, K.launch_count() - before,
                      keep=(arena, ctx, handles, bts, want))

    def capture_all(self) -> int:
        """Capture every bucket now (largest first), so that no step of a served request pays for
        a capture; returns how many graphs were captured (``emberserve/engine.py:322-334`` captures
        at boot as well)."""
        done = 0
        for bucket in sorted(self.buckets, reverse=True):
            if bucket not in self._graphs:
                self._graphs[bucket] = self._capture(bucket)
                done += 1
        return done

    def verify_scratch(self) -> None:
        for g in self._graphs.values():
            g.keep[0].verify()

    def run(self, rows) -> torch.Tensor:
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
