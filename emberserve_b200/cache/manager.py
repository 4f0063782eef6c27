"""Bookkeeping of the cache: pages of keys and values with a block table per request,
per *group* of cache entries, and slots of fixed-size state.  Pure Python, no tensors.

Cache entries (one per layer call that keeps something) with equal needs form a group.
Every paged group has pages of its own: its own pool, its own block table per request.
A group whose entries read only a window of keys gives pages back as soon as the window
has passed them; a request that ends gives back everything.  Freed pages go to the back
of the pool and are handed out again from the front, with whatever they still contain
(``emberserve/kv/block_manager.py:69-72,132-152``: same deque discipline, same
``allocate`` / ``append_slots`` / ``free`` life cycle, reference counts kept for sharing).

State slots: a request takes one slot at admission and returns it when it ends.  A slot
is marked *fresh* when it is handed out so that the storage zeroes it before first use.
The reference has nothing of this kind (its only per-request state is the sampler's
generator); it is here for mixers that carry state of fixed size.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from emberserve_b200.parts.base import CacheNeed, FixedState, PagedKV


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots); the manager's state is unchanged."""


@dataclass(frozen=True)
class CacheGroup:
    need: CacheNeed
    entries: tuple[int, ...]  # cache entry ids, in order

    @property
    def paged(self) -> bool:
        return isinstance(self.need, PagedKV)


def plan_groups(entries: list[CacheNeed]) -> list[CacheGroup]:
    """Group cache entries by equal needs, in order of first appearance."""
    order: list[CacheNeed] = []
    members: dict[CacheNeed, list[int]] = {}
    for i, need in enumerate(entries):
        if need not in members:
            members[need] = []
            order.append(need)
        members[need].append(i)
    return [CacheGroup(n, tuple(members[n])) for n in order]


class PagePool:
    """Free list and reference counts of one group's pages."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._ref = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free pages")
        page = self._free.popleft()
        assert self._ref[page] == 0, f"page {page} on the free list is still referenced"
        self._ref[page] = 1
        return page

    def share(self, page: int) -> None:
        assert self._ref[page] > 0, "cannot share a free page"
        self._ref[page] += 1

    def give(self, page: int) -> None:
        assert self._ref[page] > 0, f"page {page} freed twice"
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)

    def ref_count(self, page: int) -> int:
        return self._ref[page]

    def free_pages(self) -> list[int]:
        return list(self._free)

    def reset(self) -> None:
        self._free = deque(range(self.num_pages))
        self._ref = [0] * self.num_pages


@dataclass
class _Sequence:
    num_tokens: int  # token slots reserved (positions [0, num_tokens))
    committed: int = 0  # tokens whose keys and values are in the cache
    tables: list[list[int]] = field(default_factory=list)  # per paged group; -1 = given back
    released: list[int] = field(default_factory=list)  # per paged group: leading pages given back
    slot: int = -1
    # The tables once more as int32 arrays (given-back pages as 0, a valid id that is never
    # read), kept in step with `tables`, so that a step copies them without a Python loop.
    arrays: list[np.ndarray] = field(default_factory=list)

    def append_page(self, k: int, page: int) -> None:
        table = self.tables[k]
        arr = self.arrays[k]
        if len(table) >= arr.size:
            grown = np.zeros(max(8, 2 * arr.size), dtype=np.int32)
            grown[:arr.size] = arr
            self.arrays[k] = arr = grown
        arr[len(table)] = page
        table.append(page)


@dataclass
class CacheStats:
    page_size: int
    num_pages: list[int]
    num_free: list[int]
    used_token_slots: int
    num_sequences: int
    num_state_slots: int
    free_state_slots: int


class CacheManager:
    def __init__(self, groups: list[CacheGroup], num_pages: int | list[int], page_size: int,
                 num_state_slots: int = 0) -> None:
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        self.paged_groups = [i for i, g in enumerate(self.groups) if g.paged]
        self.state_groups = [i for i, g in enumerate(self.groups) if not g.paged]
        counts = num_pages if isinstance(num_pages, list) else [num_pages] * len(self.paged_groups)
        if len(counts) != len(self.paged_groups):
            raise ValueError("one page count per paged group is needed")
        self.pools = [PagePool(n) for n in counts]
        self.windows: list[int | None] = [self.groups[i].need.window for i in self.paged_groups]
        self.num_state_slots = num_state_slots if self.state_groups else 0
        self._free_slots: deque[int] = deque(range(self.num_state_slots))
        self._fresh_slots: set[int] = set()
        self._seqs: dict[int, _Sequence] = {}

    # ---- queries -------------------------------------------------------------------------
    def pages_needed(self, num_tokens: int) -> int:
        return -(-num_tokens // self.page_size)

    def has_sequence(self, seq_id: int) -> bool:
        return seq_id in self._seqs

    def num_tokens(self, seq_id: int) -> int:
        """Token slots reserved for the request."""
        return self._seqs[seq_id].num_tokens

    def committed(self, seq_id: int) -> int:
        return self._seqs[seq_id].committed

    def table(self, seq_id: int, paged_group: int) -> list[int]:
        """Page ids by page index for the request in the k-th paged group; -1 where the
        window has passed and the page was given back."""
        return self._seqs[seq_id].tables[paged_group]

    def table_array(self, seq_id: int, paged_group: int) -> np.ndarray:
        """The same table as an int32 array, with 0 where a page was given back."""
        seq = self._seqs[seq_id]
        return seq.arrays[paged_group][:len(seq.tables[paged_group])]

    def state_slot(self, seq_id: int) -> int:
        return self._seqs[seq_id].slot

    def num_free_pages(self, paged_group: int = 0) -> int:
        return self.pools[paged_group].num_free

    def can_admit(self, num_tokens: int) -> bool:
        need = self.pages_needed(num_tokens)
        if any(pool.num_free < need for pool in self.pools):
            return False
        return not self.state_groups or bool(self._free_slots)

    def can_extend(self, seq_id: int, num_tokens: int) -> bool:
        seq = self._seqs[seq_id]
        need = self.pages_needed(num_tokens)
        return all(need - len(t) <= pool.num_free for t, pool in zip(seq.tables, self.pools))

    def stats(self) -> CacheStats:
        return CacheStats(
            page_size=self.page_size,
            num_pages=[p.num_pages for p in self.pools],
            num_free=[p.num_free for p in self.pools],
            used_token_slots=sum(s.committed for s in self._seqs.values()),
            num_sequences=len(self._seqs),
            num_state_slots=self.num_state_slots,
            free_state_slots=len(self._free_slots))

    # ---- life cycle ----------------------------------------------------------------------
    def admit(self, seq_id: int, num_tokens: int) -> None:
        """Reserve pages for positions [0, num_tokens) in every paged group and take a
        state slot.  Raises OutOfPages, changing nothing, if that cannot be had."""
        assert seq_id not in self._seqs, f"request {seq_id} is already admitted"
        need = self.pages_needed(num_tokens)
        for k, pool in enumerate(self.pools):
            if pool.num_free < need:
                raise OutOfPages(f"group {k}: need {need} pages, have {pool.num_free}")
        if self.state_groups and not self._free_slots:
            raise OutOfPages("no free state slot")
        seq = _Sequence(num_tokens=num_tokens)
        for k, pool in enumerate(self.pools):
            seq.tables.append([])
            seq.arrays.append(np.zeros(max(8, need), dtype=np.int32))
            seq.released.append(0)
            for _ in range(need):
                seq.append_page(k, pool.take())
        if self.state_groups:
            seq.slot = self._free_slots.popleft()
            self._fresh_slots.add(seq.slot)
        self._seqs[seq_id] = seq

    def extend(self, seq_id: int, num_tokens: int) -> None:
        """Make room for positions up to `num_tokens` (decode: one more).  Raises
        OutOfPages leaving the request as it was (``block_manager.py:168-179``)."""
        seq = self._seqs[seq_id]
        if num_tokens <= seq.num_tokens:
            return
        need = self.pages_needed(num_tokens)
        for k, (table, pool) in enumerate(zip(seq.tables, self.pools)):
            if need - len(table) > pool.num_free:
                raise OutOfPages(f"group {k}: need {need - len(table)} pages, have {pool.num_free}")
        for k, (table, pool) in enumerate(zip(seq.tables, self.pools)):
            while len(table) < need:
                seq.append_page(k, pool.take())
        seq.num_tokens = num_tokens
        # A page that a window passed before it was ever needed is given back at once.
        self._release_passed(seq)

    def commit(self, seq_id: int, computed: int) -> None:
        """Record that keys and values of positions [0, computed) are in the cache, and
        give back the pages that no later query of a windowed group can read."""
        seq = self._seqs[seq_id]
        assert seq.committed <= computed <= seq.num_tokens, (seq.committed, computed, seq.num_tokens)
        seq.committed = computed
        self._release_passed(seq)

    def _release_passed(self, seq: _Sequence) -> None:
        for k, window in enumerate(self.windows):
            if window is None:
                continue
            # The next query stands at position >= committed and reads keys > committed - window.
            first_needed = max(0, seq.committed - window + 1)
            upto = min(first_needed // self.page_size, len(seq.tables[k]))
            table = seq.tables[k]
            for i in range(seq.released[k], upto):
                self.pools[k].give(table[i])
                table[i] = -1
                seq.arrays[k][i] = 0
            seq.released[k] = max(seq.released[k], upto)

    def release(self, seq_id: int) -> None:
        """Give back everything the request holds.  Idempotent."""
        seq = self._seqs.pop(seq_id, None)
        if seq is None:
            return
        for table, pool in zip(seq.tables, self.pools):
            for page in table:
                if page >= 0:
                    pool.give(page)
        if seq.slot >= 0:
            self._fresh_slots.discard(seq.slot)
            self._free_slots.append(seq.slot)

    def take_fresh_slots(self) -> list[int]:
        """Slots handed out since the last call: the storage zeroes them before use."""
        fresh = sorted(self._fresh_slots)
        self._fresh_slots.clear()
        return fresh

    def reset(self) -> None:
        for pool in self.pools:
            pool.reset()
        self._free_slots = deque(range(self.num_state_slots))
        self._fresh_slots.clear()
        self._seqs.clear()

    # ---- self-check (tests) ----------------------------------------------------------------
    def check(self) -> None:
        """Every page is free or held exactly as often as its reference count says; no
        page is lost; no slot is held twice."""
        for k, pool in enumerate(self.pools):
            held: dict[int, int] = {}
            for seq in self._seqs.values():
                for page in seq.tables[k]:
                    if page >= 0:
                        held[page] = held.get(page, 0) + 1
            free = pool.free_pages()
            assert len(free) == len(set(free)), f"group {k}: a page is on the free list twice"
            assert not set(free) & set(held), f"group {k}: a held page is on the free list"
            assert len(free) + len(held) == pool.num_pages, f"group {k}: a page is lost"
            for page, n in held.items():
                assert pool.ref_count(page) == n, f"group {k}: page {page} held {n}x, ref {pool.ref_count(page)}"
        slots = [s.slot for s in self._seqs.values() if s.slot >= 0]
        assert len(slots) == len(set(slots)), "a state slot is held twice"
        assert len(slots) + len(self._free_slots) == self.num_state_slots, "a state slot is lost"
