"""Slots for per-request state of fixed size.

Every admitted request holds one slot; a mixer that keeps state (declared with a
``StateSlot`` record) gets a device tensor ``[num_slots, *shape]`` and indexes it with the
step's slot ids.  This architecture's mixers declare none, so the slot is an index and
nothing else.  Slot 0 is never handed out: padded rows of a captured decode step use it.
"""
from __future__ import annotations

from typing import Dict, List


class OutOfSlots(RuntimeError):
    pass


class SlotAllocator:
    def __init__(self, max_requests: int):
        if max_requests < 1:
            raise ValueError("at least one request slot is needed")
        self.max_requests = max_requests
        self._free: List[int] = list(range(max_requests, 0, -1))    # slots 1..max_requests
        self._owner: Dict[object, int] = {}

    @property
    def num_slots(self) -> int:
        """Rows a state tensor needs (slot 0 included)."""
        return self.max_requests + 1

    @property
    def available(self) -> int:
        return len(self._free)

    def acquire(self, req) -> int:
        if req in self._owner:
            raise ValueError(f"request {req!r} already holds slot {self._owner[req]}")
        if not self._free:
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        s = self._free.pop()
        self._owner[req] = s
        return s

    def release(self, req) -> int:
        if req not in self._owner:
            raise ValueError(f"request {req!r} holds no slot")
        s = self._owner.pop(req)
        self._free.append(s)
        return s

    def slot_of(self, req) -> int:
        return self._owner[req]

    def holders(self):
        return dict(self._owner)
