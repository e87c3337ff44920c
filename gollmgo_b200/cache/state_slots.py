"""Slots for per-request state of fixed size.

A request takes one slot index at admission and gives it back when it ends; every
fixed-state buffer of the model is indexed by it (``buffer[slot]``).  The Llama
decoder keeps no such state, so it owns no buffers here, but the slot index is
still part of every batch: a mixer with recurrent state finds its rows by it.
The reference has nothing of the kind.
"""
from __future__ import annotations

from typing import Dict, List


class OutOfStateSlots(RuntimeError):
    pass


class StateSlots:
    def __init__(self, max_requests: int):
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        self.max_requests = max_requests
        self._free: List[int] = list(range(max_requests - 1, -1, -1))
        self._held: Dict[int, bool] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfStateSlots(f"all {self.max_requests} request slots are taken")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._held:
            raise RuntimeError(f"state slot {slot} given back twice")
        del self._held[slot]
        self._free.append(slot)

    def held(self) -> List[int]:
        return sorted(self._held)
