"""The cache manager: pages for every group, a slot per request, and the device storage.

Lifecycle of a request: ``admit`` (a slot), then before each step ``reserve`` (pages in
every group for the positions the step touches; all or nothing), after the step ``commit``
(the new length; window groups give passed pages back), at the end ``release`` (everything
back).  Host-side logic needs no GPU: with ``device=None`` no storage is allocated and only
the bookkeeping runs.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .groups import NO_PAGE, CacheGroup, CacheNeed, PagedKV, StateSlot
from .pages import OutOfPages
from .slots import OutOfSlots, SlotAllocator


class KVView:
    """What a mixer sees of its cache: its pages and the group whose block table indexes them."""

    def __init__(self, group_index: int, k_pages, v_pages, page_size: int):
        self.group_index = group_index
        self.k_pages, self.v_pages, self.page_size = k_pages, v_pages, page_size


class StateView:
    """A state-keeping mixer's tensor ``[num_slots, *shape]``; index it with the step's slot ids."""

    def __init__(self, state):
        self.state = state


class CacheManager:
    def __init__(self, needs: Sequence[object], num_pages: int, page_size: int, max_requests: int,
                 max_positions: int, dtype: torch.dtype = torch.bfloat16, device=None,
                 pages_per_group: Optional[Dict[int, int]] = None):
        """``needs[c]`` is what cache ``c`` asks for: a ``PagedKV``, a ``StateSlot`` or None.

        ``num_pages`` is the number of usable pages of every group (one more, the null page,
        is added); ``pages_per_group`` overrides it by group index.
        """
        if page_size < 1:
            raise ValueError("page size must be positive")
        self.page_size = page_size
        self.max_positions = max_positions
        self.max_blocks = (max_positions + page_size - 1) // page_size
        self.dtype, self.device = dtype, device
        self.slots = SlotAllocator(max_requests)
        self.groups: List[CacheGroup] = []
        self.views: List[object] = [None] * len(needs)
        self.lengths: Dict[object, int] = {}
        self._state_tensors: List[torch.Tensor] = []
        # request -> positions that every group has pages for already (a step within them asks the groups nothing:
        # fifteen of sixteen decode steps with pages of 16)
        self._room: Dict[object, int] = {}

        # Needs with equal group keys share a group; a need without a key (per-request state) gets storage of its own.
        # What each kind of need provides is the need's own business (``CacheNeed`` in groups.py).
        by_key: Dict[object, List[int]] = {}
        for c, need in enumerate(needs):
            if need is not None and need.group_key() is not None:
                by_key.setdefault(need.group_key(), []).append(c)
        for gi, (key, ids) in enumerate(by_key.items()):
            need = needs[ids[0]]
            n = (pages_per_group or {}).get(gi, num_pages)
            self.groups.append(need.make_group(ids, n + 1, page_size, self.max_blocks))
            storage = need.make_storage(len(ids), n + 1, page_size, self.slots.num_slots, dtype, device)
            for i, c in enumerate(ids):
                self.views[c] = need.make_view(storage, i, gi, page_size)
        for c, need in enumerate(needs):
            if need is not None and need.group_key() is None:
                storage = need.make_storage(1, 0, page_size, self.slots.num_slots, dtype, device)
                if storage is not None and hasattr(storage, "zero_"):
                    self._state_tensors.append(storage)
                self.views[c] = need.make_view(storage, 0, -1, page_size)

    # ---- requests ------------------------------------------------------------------------
    def admit(self, req) -> int:
        slot = self.slots.acquire(req)         # raises OutOfSlots
        self.lengths[req] = 0
        for st in self._state_tensors:
            st[slot].zero_()
        return slot

    def is_live(self, req) -> bool:
        return req in self.lengths

    def length(self, req) -> int:
        return self.lengths[req]

    def pages_needed(self, req, new_len: int) -> List[int]:
        if new_len <= self._room.get(req, 0):
            return [0] * len(self.groups)
        start = self.lengths.get(req, 0)
        return [g.pages_needed(req, start, new_len) for g in self.groups]

    def can_reserve(self, wants: Dict[object, int]) -> bool:
        """Would ``reserve`` succeed for all of ``{request: new_len}`` together?"""
        need = [0] * len(self.groups)
        room = self._room
        for req, new_len in wants.items():
            if new_len <= room.get(req, 0):
                continue
            for gi, n in enumerate(self.pages_needed(req, new_len)):
                need[gi] += n
        return all(n <= g.pool.available for n, g in zip(need, self.groups))

    def reserve(self, req, new_len: int) -> None:
        """Pages in every group for a step that takes ``req`` from its length to ``new_len``."""
        if req not in self.lengths:
            raise KeyError(f"request {req!r} was not admitted")
        if new_len > self.max_positions:
            raise ValueError(f"request {req!r}: {new_len} positions exceed the maximum of {self.max_positions}")
        if new_len <= self._room.get(req, 0):
            return
        start = self.lengths[req]
        done = []
        try:
            for g in self.groups:
                done.append((g, g.reserve(req, start, new_len)))
        except OutOfPages:
            for g, pages in done:
                g.give_back(req, pages)
            raise
        self._room[req] = min((len(g.tables[req]) for g in self.groups), default=0) * self.page_size if self.groups else self.max_positions

    def commit(self, req, new_len: int) -> None:
        self.lengths[req] = new_len
        for g in self.groups:
            g.trim(req, new_len)

    def truncate(self, req, new_len: int) -> None:
        """Go back to ``new_len`` cached positions (new_len <= the current length)."""
        if new_len > self.lengths[req]:
            raise ValueError(f"request {req!r} holds {self.lengths[req]} positions, cannot truncate to {new_len}")
        for g in self.groups:
            g.truncate(req, new_len)
        self.lengths[req] = new_len
        self._room[req] = min((len(g.tables.get(req, ())) for g in self.groups), default=0) * self.page_size if self.groups else self.max_positions

    def release(self, req) -> None:
        if req not in self.lengths:
            raise KeyError(f"request {req!r} is not live")
        for g in self.groups:
            g.release(req)
        self.slots.release(req)
        del self.lengths[req]
        self._room.pop(req, None)

    # ---- what a step uploads ----------------------------------------------------------------
    def block_table_rows(self, group_index: int, reqs: Sequence[object], out: np.ndarray) -> None:
        """Fill ``out[i, :]`` (int32, ``[len(reqs), max_blocks]``) with request i's pages."""
        g = self.groups[group_index]
        for i, r in enumerate(reqs):
            row = g.row(r)
            if row is None:
                out[i].fill(NO_PAGE)
            else:
                out[i] = row

    def slot_ids(self, reqs: Sequence[object]) -> List[int]:
        return [self.slots.slot_of(r) for r in reqs]

    # ---- accounting ------------------------------------------------------------------------
    def stats(self) -> dict:
        return {
            "live_requests": len(self.lengths),
            "groups": [{"name": g.name, "pages_in_use": g.pool.in_use, "pages_free": g.pool.available,
                        "high_water": g.pool.high_water} for g in self.groups],
        }

    def check_invariants(self) -> None:
        """No page lost, none held twice: every page is free or in exactly one table."""
        for g in self.groups:
            seen = {}
            for req, table in g.tables.items():
                for p in table:
                    if p == NO_PAGE:
                        continue
                    if p in seen:
                        raise AssertionError(f"{g.name}: page {p} held by {seen[p]!r} and {req!r}")
                    seen[p] = req
            held = set(g.pool.held_pages())
            if held != set(seen):
                raise AssertionError(f"{g.name}: pool says {sorted(held)} are out, tables hold {sorted(seen)}")
            if g.pool.in_use + g.pool.available != g.pool.capacity:
                raise AssertionError(f"{g.name}: a page is lost")
            for req, room in self._room.items():
                table = g.tables.get(req, [])
                last = (room + self.page_size - 1) // self.page_size
                first = max(g._first_needed_block(self.lengths.get(req, 0)), g.first_block.get(req, 0))
                if last > len(table) or any(p == NO_PAGE for p in table[first:last]):
                    raise AssertionError(f"{g.name}: {req!r} is said to have pages for {room} positions and has not")
            for req, table in g.tables.items():
                row = g.row(req)
                mirror = [] if row is None else row.tolist()
                if mirror[:len(table)] != table and any(p != NO_PAGE for p in table):
                    raise AssertionError(f"{g.name}: the row of {req!r} differs from its table")
                if any(p != NO_PAGE for p in mirror[len(table):]):
                    raise AssertionError(f"{g.name}: the row of {req!r} holds pages beyond its table")
