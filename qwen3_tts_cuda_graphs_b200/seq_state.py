"""Per-sequence state of the sequence models: slots, position counters, caches that grow with the position and fixed-size carries.

A model declares what each of its layers keeps between steps as `StateSpec`s:
  * kind "append": one row per position (`rows` = capacity in positions): an attention's cached latents / keys / values;
  * kind "carry":  a fixed block that a step reads and replaces: the last inputs of a causal convolution, a recurrent state.
A carry is double-buffered (`cur`, `next`): the step's kernels read `cur` and write `next`, and the step's last op
(FQ3C_COMMIT, include/fq3_codec.h) copies every `next` to its `cur` and advances the slot's device position counter in one
launch.  All addresses are fixed for the life of the manager, so a captured op list replays at any position of any request
that later occupies the slot.  A slot is handed to one request at a time; releasing it gives everything back, and acquiring
zeroes the carries and the counter (a cache needs no clearing: rows at or beyond the counter are never read).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class StateSpec:
    name: str
    kind: str                 # "append" | "carry"
    cols: int
    rows: int = 1             # carry: rows of the block; append: ignored (capacity comes from the manager)
    dtype: torch.dtype = torch.float32


class SlotState:
    def __init__(self, index: int, specs: List[StateSpec], max_pos: int, device):
        self.index = index
        self.max_pos = max_pos
        self.length = 0                      # host mirror of the device counter
        self.owner: Optional[object] = None
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.cur: Dict[str, torch.Tensor] = {}
        self.next: Dict[str, torch.Tensor] = {}
        table = []
        for s in specs:
            if s.kind == "append":
                self.cur[s.name] = torch.zeros(max_pos, s.cols, dtype=s.dtype, device=device)
            elif s.kind == "carry":
                if s.rows <= 0:
                    continue
                a = torch.zeros(s.rows, s.cols, dtype=s.dtype, device=device)
                b = torch.zeros(s.rows, s.cols, dtype=s.dtype, device=device)
                self.cur[s.name], self.next[s.name] = a, b
                table.append([a.data_ptr(), b.data_ptr(), a.numel() * a.element_size()])
            else:
                raise ValueError(f"unknown state kind {s.kind!r}")
        self.n_commit = len(table)
        # (dst, src, bytes) rows of the step-closing commit; one dummy row keeps the launch shape valid for stateless models
        self.commit = torch.tensor(table or [[0, 0, 0]], dtype=torch.int64, device=device)

    def reset(self):
        for name, t in self.next.items():
            t.zero_()
            self.cur[name].zero_()
        self.pos.zero_()
        self.length = 0

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self.cur.values()) + list(self.next.values()))


class SequenceStateManager:
    """Slots of `max_pos` positions each.  Slots are created on demand up to `max_slots` and reused after release."""

    def __init__(self, specs: List[StateSpec], max_pos: int, device, max_slots: int = 1):
        names = [s.name for s in specs]
        if len(set(names)) != len(names):
            raise ValueError("state names must be unique")
        self.specs, self.max_pos, self.device, self.max_slots = list(specs), int(max_pos), device, int(max_slots)
        self.slots: List[SlotState] = []
        self.by_owner: Dict[object, SlotState] = {}

    def acquire(self, owner) -> SlotState:
        if owner in self.by_owner:
            raise KeyError(f"request {owner!r} already holds a slot")
        slot = next((s for s in self.slots if s.owner is None), None)
        if slot is None:
            if len(self.slots) >= self.max_slots:
                raise RuntimeError(f"all {self.max_slots} sequence slots are in use")
            slot = SlotState(len(self.slots), self.specs, self.max_pos, self.device)
            self.slots.append(slot)
        slot.reset()
        slot.owner = owner
        self.by_owner[owner] = slot
        return slot

    def get(self, owner) -> Optional[SlotState]:
        return self.by_owner.get(owner)

    def release(self, owner) -> None:
        slot = self.by_owner.pop(owner, None)
        if slot is not None:
            slot.owner = None

    def reserve(self, slot: SlotState, n_tokens: int) -> int:
        """Host-side bookkeeping of a step of n_tokens: returns the position of its first token."""
        if slot.length + n_tokens > slot.max_pos:
            raise RuntimeError(f"sequence of {slot.length + n_tokens} positions exceeds the slot capacity {slot.max_pos}")
        start = slot.length
        slot.length += n_tokens
        return start

    def free_slots(self) -> int:
        return self.max_slots - len(self.by_owner)
