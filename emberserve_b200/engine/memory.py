"""How the device memory is divided between the cache and everything a step allocates.

The cache is sized from the memory that is free once the weights are resident
(``emberserve/engine.py:141-153``): ``free * utilization - reserve``, in whole pages.  The
reserve is what the engine will still allocate AFTER the cache exists, at its busiest
step; a reserve that is too small fails late, when the largest CUDA graph is captured or
the first full-budget prompt portion runs.  The reference reserves a workspace of 1 GiB,
the gate/up activations of one prompt portion and the logits of the largest decode batch
(``emberserve/engine.py:121-139``).  Here the terms are those of this engine:

* ``workspace``: 1 GiB for cuBLAS workspaces, the graphs' memory pool, the allocator's
  slack and the sampler's buffers;
* ``step_scratch``: the scratch buffers of the largest eager step, ``max_step_tokens``
  rows of every buffer a block asks for (`Decoder.scratch_bytes_per_token`: the 32-bit
  residual, and the widest block's activations);
* ``step_logits``: float32 logits of ``max_logit_rows`` rows of an eager step;
* ``graph_scratch`` and ``graph_logits``: the same for the ONE arena that all captured
  decode graphs share, ``graph_rows`` rows (the buckets never run at the same time);
* ``state``: the slots of fixed-size state, if a mixer keeps any.
"""

from __future__ import annotations

from dataclasses import dataclass

WORKSPACE_BYTES = 1 << 30


@dataclass(frozen=True)
class MemoryPlan:
    free_bytes: int
    utilization: float
    workspace: int
    step_scratch: int
    step_logits: int
    graph_scratch: int
    graph_logits: int
    state: int
    bytes_per_page: int
    num_pages: int

    @property
    def reserve(self) -> int:
        return (self.workspace + self.step_scratch + self.step_logits + self.graph_scratch
                + self.graph_logits + self.state)

    @property
    def cache_bytes(self) -> int:
        return self.num_pages * self.bytes_per_page


def plan_memory(*, free_bytes: int, utilization: float, bytes_per_page: int, scratch_bytes_per_token: int,
                vocab_size: int, max_step_tokens: int, max_logit_rows: int, graph_rows: int,
                state_bytes: int = 0, reserve_override: int | None = None) -> MemoryPlan:
    """Pages of the cache for `free_bytes` of free device memory (weights already resident).
    `graph_rows` = 0 if no CUDA graphs will be captured.  With `reserve_override` that many
    bytes are kept free instead of the computed terms (they are still reported)."""
    plan = dict(
        workspace=WORKSPACE_BYTES,
        step_scratch=max_step_tokens * scratch_bytes_per_token,
        step_logits=max_logit_rows * vocab_size * 4,
        graph_scratch=graph_rows * scratch_bytes_per_token,
        graph_logits=graph_rows * vocab_size * 4,
        state=state_bytes)
    reserve = sum(plan.values()) if reserve_override is None else reserve_override
    budget = int(free_bytes * utilization) - reserve
    pages = max(0, budget // bytes_per_page) if bytes_per_page > 0 else 0
    return MemoryPlan(free_bytes=free_bytes, utilization=utilization, bytes_per_page=bytes_per_page,
                      num_pages=pages, **plan)
