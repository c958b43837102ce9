"""Slots for per-request state of fixed size.

Every live request holds one slot, whether or not any layer keeps such state: the slot
index is what the step passes to the parts (`StepContext.state_slots`).  A layer whose
mixer declares a `FixedStateNeed` gets a tensor [max_live, *shape]; the row of a slot is
cleared when a request takes it.  The reference's counterpart is the host-side slot
of a request (jllm/engine/runtime.py:12-35); it keeps no device state per request.
"""

from __future__ import annotations

import torch


class StateSlots:
    def __init__(self, max_live: int):
        self.max_live = max_live
        self.free = list(range(max_live - 1, -1, -1))   # pop() gives the lowest index first
        self.held: set[int] = set()
        self.tensors: dict[int, torch.Tensor] = {}      # layer -> [max_live, *shape]

    def add_layer(self, layer: int, shape, dtype, device) -> torch.Tensor:
        t = torch.zeros((self.max_live, *shape), dtype=dtype, device=device)
        self.tensors[layer] = t
        return t

    @property
    def num_free(self) -> int:
        return len(self.free)

    def take(self) -> int:
        if not self.free:
            raise RuntimeError("no free state slot")
        s = self.free.pop()
        self.held.add(s)
        for t in self.tensors.values():
            t[s].zero_()
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self.held:
            raise RuntimeError(f"state slot {slot} given back without being held")
        self.held.remove(slot)
        self.free.append(slot)
        self.free.sort(reverse=True)

    def bytes_per_request(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.tensors.values())
