"""Slots for fixed-size per-request state.

The reference has no such thing (its one architecture family keeps only keys and values).
Every live request holds one slot, whether or not a mixer of the model keeps state: the slot
id is also the request's row in the persistent block-table mirrors.  A mixer that declares a
StateNeed gets a tensor [slots + 1, *shape]; a request's row is zeroed when it claims the slot
(also after preemption, since recomputation starts again at position 0).  Slot 0 is scratch
for padding rows."""
from __future__ import annotations


class StateSlots:
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots, 0, -1))       # pop() gives 1, 2, ...
        self._held = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def claim(self):
        if not self._free:
            return None
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise RuntimeError(f"state slot {slot} released twice")
        self._held.remove(slot)
        self._free.append(slot)
