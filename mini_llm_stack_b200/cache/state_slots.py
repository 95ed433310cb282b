"""Slots for per-request state of fixed size.

The reference has no layer with such state.  A mixer that keeps a fixed amount
per request (a recurrent state, a convolution tail) declares ``FixedState``;
each running request then holds one slot id, the same in every such group, and
the step hands the mixer ``state_slot[R]``.  A slot is zeroed when it is claimed.
"""

from __future__ import annotations


class SlotPoolError(RuntimeError):
    pass


class StateSlotPool:
    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._owner = [None] * self.num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def claim(self, owner) -> int | None:
        if not self._free:
            return None
        s = self._free.pop()
        if self._owner[s] is not None:
            raise SlotPoolError(f"slot {s} was free but is owned")
        self._owner[s] = owner
        return s

    def release(self, slot: int, owner) -> None:
        if not (0 <= slot < self.num_slots) or self._owner[slot] is None:
            raise SlotPoolError(f"slot {slot} is released twice or unknown")
        if self._owner[slot] != owner:
            raise SlotPoolError(f"slot {slot} belongs to {self._owner[slot]!r}")
        self._owner[slot] = None
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise SlotPoolError("a slot is on the free list twice")
        for s in range(self.num_slots):
            if (s in free) == (self._owner[s] is not None):
                raise SlotPoolError(f"slot {s} is lost or held twice")
