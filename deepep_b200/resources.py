"""Slot and handle life cycle of the V1 ``Buffer``.

A buffer owns a small number of *slots*; one dispatch occupies one slot until its combine has finished (or the
handle is released), and a handle is only honoured while the slot still belongs to it.  The slot counts its uses
(*generation*), so a stale handle -- one whose slot has meanwhile served another dispatch -- is refused instead of
combining with foreign routing state.

Parity: ``deep_ep/backends/direct/resources.py:11-184`` of the reference (``SlotState`` FREE -> ACQUIRED ->
DISPATCH_IN_FLIGHT -> DISPATCH_READY -> COMBINE_IN_FLIGHT -> RELEASABLE -> FREE, generation-checked ``Handle``).
"""
from __future__ import annotations

import enum
from typing import List, Optional, Tuple

import torch


class SlotState(enum.Enum):
    FREE = "free"
    ACQUIRED = "acquired"
    DISPATCH_IN_FLIGHT = "dispatch_in_flight"
    DISPATCH_READY = "dispatch_ready"
    COMBINE_IN_FLIGHT = "combine_in_flight"
    RELEASABLE = "releasable"


_NEXT = {
    SlotState.FREE: (SlotState.ACQUIRED,),
    SlotState.ACQUIRED: (SlotState.DISPATCH_IN_FLIGHT, SlotState.FREE),
    SlotState.DISPATCH_IN_FLIGHT: (SlotState.DISPATCH_READY, SlotState.FREE),
    # a handle may serve several cached dispatches and several combines (forward and backward) before it is released
    SlotState.DISPATCH_READY: (SlotState.COMBINE_IN_FLIGHT, SlotState.DISPATCH_IN_FLIGHT, SlotState.RELEASABLE, SlotState.FREE),
    SlotState.COMBINE_IN_FLIGHT: (SlotState.RELEASABLE, SlotState.DISPATCH_READY),
    SlotState.RELEASABLE: (SlotState.FREE, SlotState.COMBINE_IN_FLIGHT, SlotState.DISPATCH_IN_FLIGHT),
}


class Slot:
    def __init__(self, index: int):
        self.index, self.state, self.generation = index, SlotState.FREE, 0

    def move(self, new: SlotState) -> None:
        if new not in _NEXT[self.state]:
            raise RuntimeError(f"slot {self.index}: illegal transition {self.state.value} -> {new.value}")
        if new is SlotState.ACQUIRED:
            self.generation += 1
        self.state = new


class SlotPool:
    """The slots of one buffer.  ``acquire`` prefers a free slot and otherwise recycles the oldest releasable one."""

    def __init__(self, count: int = 4):
        self.slots: List[Slot] = [Slot(i) for i in range(count)]
        self._order: List[int] = []

    def acquire(self) -> Slot:
        for s in self.slots:
            if s.state is SlotState.FREE:
                s.move(SlotState.ACQUIRED)
                self._order.append(s.index)
                return s
        for index in list(self._order):
            s = self.slots[index]
            if s.state in (SlotState.RELEASABLE, SlotState.DISPATCH_READY):     # oldest finished dispatch gives way
                self._order.remove(index)
                s.move(SlotState.FREE)
                s.move(SlotState.ACQUIRED)
                self._order.append(index)
                return s
        raise RuntimeError("every slot of this buffer has an operation in flight; wait for one to finish")

    def release(self, slot: Slot) -> None:
        if slot.state is not SlotState.FREE:
            slot.state = SlotState.FREE
        if slot.index in self._order:
            self._order.remove(slot.index)


class Handle(tuple):
    """The V1 dispatch handle: upstream's six tensors ``(rank_prefix_matrix, channel_prefix_matrix,
    recv_channel_prefix_matrix, recv_src_idx, is_token_in_rank, send_head)`` plus the slot it occupies.

    * ``rank_prefix_matrix [P, P]``: tokens that sources ``0..i`` send to rank ``j`` (inclusive prefix over sources);
    * ``channel_prefix_matrix [P, C]``: this rank's tokens sent to rank ``j`` before 64-token chunk ``c`` (a chunk plays
      the role of upstream's channel);
    * ``recv_channel_prefix_matrix [P, C + 1]``: received rows of source ``i`` before its chunk ``c``;
    * ``recv_src_idx [R]``: token index at its source of every received row;
    * ``is_token_in_rank [T, P]``; ``send_head [T, P]``: row index of token ``t`` at rank ``j`` (-1: not sent).
    """

    def __new__(cls, tensors: Tuple[torch.Tensor, ...], slot: Optional[Slot], elastic_handle):
        self = super().__new__(cls, tensors)
        self.slot, self.generation = slot, (slot.generation if slot is not None else 0)
        self.elastic = elastic_handle              # the routing plan the kernels use
        return self

    @property
    def topk_idx(self):
        return self.elastic.topk_idx

    def check_live(self) -> None:
        if self.slot is not None and (self.slot.generation != self.generation or self.slot.state is SlotState.FREE):
            raise RuntimeError("stale handle: its slot has been released or reused by a later dispatch")


__all__ = ["Handle", "Slot", "SlotPool", "SlotState"]
