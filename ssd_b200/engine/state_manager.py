"""StateSlotManager — host bookkeeping of the recurrent-state pool of a hybrid model: one fixed-size slot per live
sequence, handed out on admission and given back when the sequence finishes or is preempted (the counterpart of
BlockManager for layers whose memory does not grow with the sequence).  A slot is never cleared on the device: the
kernels ignore its content for a sequence that starts at position 0."""
from __future__ import annotations

from collections import deque


class StateSlotManager:
    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("state pool has no slots")
        self.n_slots = n_slots
        self.free_slots: deque[int] = deque(range(n_slots))
        self.owner: dict[int, int] = {}  # slot -> seq_id

    def can_allocate(self) -> bool:
        return bool(self.free_slots)

    def allocate(self, seq) -> int:
        if seq.state_slot >= 0:
            return seq.state_slot
        if not self.free_slots:
            raise RuntimeError("out of recurrent-state slots")
        slot = self.free_slots.popleft()
        self.owner[slot] = seq.seq_id
        seq.state_slot = slot
        return slot

    def free(self, seq) -> None:
        slot = seq.state_slot
        if slot < 0:
            return
        assert self.owner.pop(slot) == seq.seq_id
        self.free_slots.append(slot)
        seq.state_slot = -1
