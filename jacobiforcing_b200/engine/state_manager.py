"""StateSlotManager — bookkeeping of recurrent-state slots, the companion of BlockManager for models whose layers carry
a state from token to token (convolution tails, scan states, delta-rule matrices).  A live request owns exactly one slot
on every such layer; the slot is handed back when the request finishes or is preempted and is reused WITHOUT clearing:
the kernels take the empty state for a request whose first token sits at position 0, whatever the slot held before."""
from __future__ import annotations

from collections import deque

from .sequence import Sequence


class StateSlotManager:
    def __init__(self, num_slots: int):
        assert num_slots > 0
        self.num_slots = num_slots
        self.free_slots = deque(range(num_slots))
        self.owner = {}                       # slot -> seq_id

    def can_allocate(self) -> bool:
        return bool(self.free_slots)

    def allocate(self, seq: Sequence) -> int:
        if getattr(seq, "state_slot", -1) >= 0:
            return seq.state_slot
        if not self.free_slots:
            raise RuntimeError("out of recurrent-state slots")
        slot = self.free_slots.popleft()
        self.owner[slot] = seq.seq_id
        seq.state_slot = slot
        return slot

    def deallocate(self, seq: Sequence) -> None:
        slot = getattr(seq, "state_slot", -1)
        if slot >= 0:
            assert self.owner.get(slot) == seq.seq_id, "state slot released by a request that does not own it"
            del self.owner[slot]
            self.free_slots.append(slot)
            seq.state_slot = -1
