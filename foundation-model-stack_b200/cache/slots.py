"""Bookkeeping of what is held: slots (one per live sequence) and blocks of key/value storage.

Both allocators refuse to give out what is held and to take back what is not, so that a slot or block
can never be lost, held twice or freed twice without an error.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """No slot or not enough blocks are free."""


class SlotAllocator:
    def __init__(self, max_slots: int) -> None:
        if max_slots <= 0:
            raise ValueError("max_slots must be positive")
        self.max_slots = max_slots
        self._free: List[int] = list(range(max_slots - 1, -1, -1))  # pop() gives the lowest first
        self._held = [False] * max_slots

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.max_slots} slots are held")
        slot = self._free.pop()
        self._held[slot] = True
        return slot

    def free(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots) or not self._held[slot]:
            raise ValueError(f"slot {slot} is not held")
        self._held[slot] = False
        self._free.append(slot)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and self._held[slot]

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.max_slots - len(self._free)


class BlockPool:
    """Free list of block ids 0..n_blocks-1.  Blocks that were freed last are given out first, so that a
    reused block is met early in tests."""

    def __init__(self, n_blocks: int) -> None:
        if n_blocks <= 0:
            raise ValueError("n_blocks must be positive")
        self.n_blocks = n_blocks
        self._free: List[int] = list(range(n_blocks - 1, -1, -1))
        self._held = [False] * n_blocks

    def alloc(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} blocks wanted, {len(self._free)} of {self.n_blocks} free")
        out = [self._free.pop() for _ in range(count)]
        for b in out:
            self._held[b] = True
        return out

    def free(self, blocks) -> None:
        for b in blocks:
            if not (0 <= b < self.n_blocks) or not self._held[b]:
                raise ValueError(f"block {b} is not held")
            self._held[b] = False
            self._free.append(b)

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_blocks - len(self._free)
