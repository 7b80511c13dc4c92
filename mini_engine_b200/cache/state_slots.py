"""Slots of fixed size for per-request state.

The reference has none (all its per-request device state is paged keys and values).  A
mixer that carries a state of fixed size across the portions of a request (a recurrence, a
running sum) gets a slot index with the request: assigned when the request first gets
cache, returned when it ends or is preempted.  The storage behind the index belongs to the
model runner; this class only hands out indices.
"""
from __future__ import annotations


class StateSlotPool:
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise RuntimeError("no free state slot")
        s = self._free.pop()
        self._held.add(s)
        return s

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise RuntimeError(f"state slot {slot} is released but not held")
        self._held.remove(slot)
        self._free.append(slot)

    def check(self) -> None:
        if len(self._free) + len(self._held) != self.num_slots or set(self._free) & self._held:
            raise RuntimeError("state slots lost or held twice")
