"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a
token budget, decodes, finishes and frees.  It decides; it touches no tensor.

Behaviour follows ``emberserve/sched/scheduler.py``:

* two queues: ``waiting`` (FIFO; preempted requests return to its FRONT) and ``running``
  in admission order (``:73-75,359``);
* admission looks at the head of ``waiting`` only, never past it; it needs a free place
  among ``max_num_seqs`` and pages for the request's WHOLE history, even if only a
  portion of it is computed in this step (``:162-197,311-336``);
* chunked mode (``:253-344``): every step first gives one token to every running request
  whose prompt is done, then spends what is left of ``max_num_batched_tokens`` on
  portions of running requests that are still in their prompt (oldest first), then on
  new requests; decode tokens are never crowded out;
* unchunked mode (``:140-238``): a step is either whole prompts or one token for every
  running request;
* when a decode token finds no page, the YOUNGEST running request is preempted: its pages
  are freed, it keeps its generated tokens and goes to the front of ``waiting`` to be
  recomputed; if the youngest is the request itself, it waits (``:210-238,352-360``).
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from emberserve_b200.cache.manager import CacheManager, OutOfPages
from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.engine.request import FinishReason, Request, RequestState


@dataclass
class SchedulerOutput:
    scheduled: list[Request] = field(default_factory=list)  # rows of the step, in order
    query_lens: list[int] = field(default_factory=list)  # tokens each row computes
    # True where the row computes the request's last outstanding token, so a token is
    # sampled for it; False for a portion that leaves more of the prompt to do.
    prefill_complete: list[bool] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    num_decode_tokens: int = 0

    @property
    def num_tokens(self) -> int:
        return sum(self.query_lens)

    @property
    def num_prefill_tokens(self) -> int:
        return self.num_tokens - self.num_decode_tokens

    @property
    def is_empty(self) -> bool:
        return not self.scheduled

    @property
    def is_prefill(self) -> bool:
        """Some row has several tokens or stays inside its prompt (``scheduler.py:337-341``)."""
        return any(q > 1 for q in self.query_lens) or not all(self.prefill_complete)

    def add(self, req: Request, qlen: int, complete: bool) -> None:
        self.scheduled.append(req)
        self.query_lens.append(qlen)
        self.prefill_complete.append(complete)


class Scheduler:
    def __init__(self, config: EngineConfig, cache: CacheManager) -> None:
        self.config = config
        self.cache = cache
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._by_id: dict[str, Request] = {}

    # ---- queue management ------------------------------------------------------------------
    def _why_never(self, req: Request) -> str | None:
        """Why `req` could never be served, or None (the rules of ``scheduler.py:78-94``, plus the
        prompt that is larger than the whole pool)."""
        cfg, n = self.config, req.num_prompt_tokens
        smallest_pool = min(p.num_pages for p in self.cache.pools) if self.cache.pools else None
        rules = (
            (req.seq_id < 0, "the engine must assign seq_id before add_request"),
            (n == 0, "empty prompt"),
            (n >= cfg.max_model_len, f"prompt has {n} tokens, max_model_len is {cfg.max_model_len}"),
            (not cfg.enable_chunked_prefill and n > cfg.max_num_batched_tokens,
             f"prompt has {n} tokens, exceeds max_num_batched_tokens {cfg.max_num_batched_tokens}"),
            (req.request_id in self._by_id, f"duplicate request_id {req.request_id!r}"),
            (smallest_pool is not None and self.cache.pages_needed(n + 1) > smallest_pool,
             f"prompt has {n} tokens, the cache holds {(smallest_pool or 0) * self.cache.page_size}"),
        )
        return next((why for hit, why in rules if hit), None)

    def add_request(self, req: Request) -> None:
        """Put `req` at the end of the waiting queue, or refuse it with the reason."""
        why = self._why_never(req)
        if why is not None:
            raise ValueError(why)
        self._by_id[req.request_id] = req
        req.state = RequestState.WAITING
        self.waiting.append(req)

    def abort_request(self, request_id: str) -> Request | None:
        """End a request wherever it stands; None if no live request has that id."""
        req = self._by_id.get(request_id)
        if req is not None:
            self._retire(req, FinishReason.ABORT)
        return req

    def finish_request(self, req: Request, reason: FinishReason) -> None:
        if not req.is_finished:
            self._retire(req, reason)

    def _retire(self, req: Request, reason: FinishReason) -> None:
        """Out of whichever queue holds it, pages and slot back, marked finished."""
        for queue in (self.waiting, self.running):
            for i, other in enumerate(queue):  # (by identity: requests compare field by field)
                if other is req:
                    del queue[i]
                    break
        self.cache.release(req.seq_id)
        self._by_id.pop(req.request_id, None)
        req.finish_reason = reason
        req.finished_time = time.perf_counter()
        req.state = RequestState.FINISHED

    def has_unfinished_requests(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    @property
    def num_running(self) -> int:
        return len(self.running)

    def get_request(self, request_id: str) -> Request | None:
        return self._by_id.get(request_id)

    # ---- one step ------------------------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        if self.config.enable_chunked_prefill:
            return self._schedule_mixed()
        if self.waiting:
            out = self._schedule_whole_prompts()
            if not out.is_empty:
                return out
        out = SchedulerOutput()
        self._give_decode_tokens(out, skip_mid_prompt=False)
        return out

    def _outstanding(self, req: Request) -> int:
        """Reserved token slots that hold nothing yet: > 0 while the prompt (or the
        recomputation after a preemption) is under way (``scheduler.py:241-251``)."""
        return self.cache.num_tokens(req.seq_id) - req.num_computed_tokens

    def _evict_newest(self) -> Request:
        """Pages ran out: the request that was admitted last gives up everything it holds and goes
        back to the FRONT of the waiting queue, to be recomputed from its tokens
        (``scheduler.py:352-360``)."""
        victim = self.running.pop()
        self.cache.release(victim.seq_id)
        victim.reset_for_recompute()
        self.waiting.appendleft(victim)
        return victim

    def _give_decode_tokens(self, out: SchedulerOutput, skip_mid_prompt: bool) -> None:
        """One more token slot for every running request that decodes, oldest first; when the
        pool is empty the newest requests are evicted until the slot can be had, and a request
        that would have to evict itself waits instead."""
        evicted: set[int] = set()
        for req in list(self.running):
            if id(req) in evicted:  # gave its pages to an older one a moment ago
                continue
            if req.hold or (skip_mid_prompt and self._outstanding(req) > 0):
                continue
            while True:
                try:
                    self.cache.extend(req.seq_id, self.cache.num_tokens(req.seq_id) + 1)
                except OutOfPages:
                    victim = self._evict_newest()
                    out.preempted.append(victim)
                    evicted.add(id(victim))
                    if victim is req:
                        return  # nothing newer was left to evict, and nobody behind it either
                    continue
                break
            out.add(req, 1, True)
            out.num_decode_tokens += 1

    def _admit(self, req: Request, now: float) -> None:
        self.waiting.popleft()
        self.cache.admit(req.seq_id, req.num_tokens)
        req.state = RequestState.RUNNING
        if req.first_scheduled_time is None:
            req.first_scheduled_time = now
        self.running.append(req)

    def _schedule_mixed(self) -> SchedulerOutput:
        out = SchedulerOutput()
        self._give_decode_tokens(out, skip_mid_prompt=True)
        budget = self.config.max_num_batched_tokens - out.num_tokens
        decoding = {id(r) for r in out.scheduled}
        for req in self.running:  # still inside their prompts, oldest first
            if budget <= 0:
                break
            if id(req) in decoding:
                continue
            left = self._outstanding(req)
            if left <= 0:
                continue
            take = min(left, budget)
            out.add(req, take, take == left)
            budget -= take
        now = time.perf_counter()
        while self.waiting and budget > 0:
            req = self.waiting[0]
            if len(self.running) >= self.config.max_num_seqs or not self.cache.can_admit(req.num_tokens):
                break
            self._admit(req, now)
            left = self._outstanding(req)
            take = min(left, budget)
            out.add(req, take, take == left)
            budget -= take
        return out

    def _schedule_whole_prompts(self) -> SchedulerOutput:
        out = SchedulerOutput()
        used = 0
        now = time.perf_counter()
        while self.waiting:
            req = self.waiting[0]
            n = req.num_tokens
            if len(self.running) >= self.config.max_num_seqs:
                break
            # Over the budget it waits for the next step, unless it is alone: a preempted
            # request recomputing prompt + output may exceed the budget and must still run
            # (``scheduler.py:172-178``).
            if used + n > self.config.max_num_batched_tokens and out.scheduled:
                break
            if not self.cache.can_admit(n):
                break
            self._admit(req, now)
            out.add(req, n, True)
            used += n
        return out
