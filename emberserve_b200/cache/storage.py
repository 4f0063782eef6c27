"""Device memory of the cache: pages of keys and values per paged group, state per slot.

A paged group with E entries holds one tensor ``[E, 2, num_pages, kv_heads, page_size,
head_dim]`` (2 = keys, values), so the keys of one (page, KV head) are one contiguous tile
of ``page_size * head_dim`` elements.  The reference keeps ``[num_blocks, block_size,
kv_heads, head_dim]`` per layer (``emberserve/kv/cache.py:30-34``); the geometry (pages of
``block_size`` token slots, slot = page * page_size + offset) is the same.  Contents are
never cleared when pages change hands.  A state group holds ``[E, num_slots, *shape]``,
zeroed slot by slot when a slot is handed to a new request.
"""

from __future__ import annotations

import torch

from emberserve_b200.cache.manager import CacheGroup
from emberserve_b200.parts.base import FixedState, FixedStateHandle, PagedKV, PagedKVHandle

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheStorage:
    def __init__(self, groups: list[CacheGroup], num_pages: list[int], page_size: int,
                 num_state_slots: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.groups = groups
        self.page_size = page_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.tensors: list[torch.Tensor] = []
        # entry id -> (group index, index inside the group, index among paged groups or -1)
        self.where: dict[int, tuple[int, int, int]] = {}
        paged_seen = 0
        for gi, g in enumerate(groups):
            if isinstance(g.need, PagedKV):
                n = num_pages[paged_seen]
                t = torch.zeros(len(g.entries), 2, n, g.need.num_kv_heads, page_size, g.need.head_dim,
                                dtype=dtype, device=self.device)
                for j, e in enumerate(g.entries):
                    self.where[e] = (gi, j, paged_seen)
                paged_seen += 1
            else:
                assert isinstance(g.need, FixedState)
                t = torch.zeros(len(g.entries), max(1, num_state_slots), *g.need.shape,
                                dtype=_STATE_DTYPES[g.need.dtype], device=self.device)
                for j, e in enumerate(g.entries):
                    self.where[e] = (gi, j, -1)
            self.tensors.append(t)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)

    def paged_group_of(self, entry: int) -> int:
        return self.where[entry][2]

    def zero_slots(self, slots: "list[int] | torch.Tensor") -> None:
        """Zero the state of the given slots in every state group.  `slots` may be an int32
        tensor on the device (the way a step brings them; a slot may appear more than once), so
        that the fill is an ordinary launch of the step, also inside a CUDA graph."""
        if isinstance(slots, torch.Tensor):
            if slots.numel() == 0:
                return
            idx = slots.long()
        else:
            if not slots:
                return
            idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        for g, t in zip(self.groups, self.tensors):
            if not g.paged:
                t.index_fill_(1, idx, 0)

    def handle(self, entry: int, write: bool, block_tables: list[torch.Tensor],
               slots: torch.Tensor | None) -> PagedKVHandle | FixedStateHandle:
        gi, j, pk = self.where[entry]
        need = self.groups[gi].need
        t = self.tensors[gi]
        if isinstance(need, PagedKV):
            return PagedKVHandle(k=t[j, 0], v=t[j, 1], block_tables=block_tables[pk],
                                 page_size=self.page_size, window=need.window, write=write)
        return FixedStateHandle(state=t[j], slots=slots, write=write)

    def reset(self) -> None:
        for t in self.tensors:
            t.zero_()
