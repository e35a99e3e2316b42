"""Host-side bookkeeping of the cache: pages, slots, and each sequence's length.

The reference keeps one `Session` per conversation: a position, a capacity and
flat cache rows `[layer][pos][row]` (src/model.rs:686-728; GPU: one buffer per
layer, src/cuda.rs:9945-9975), and rewinds by lowering `pos` (src/model.rs:803-806).
A batch needs the same per sequence, so the unit here is a slot: one sequence's
length and its list of pages.  Pages are `PAGE_TOKENS` positions wide; a pool
hands them out and takes them back, so memory is sized by the tokens that are
alive, not by slots x longest sequence.  Lengths are the only truth: rows past
a slot's length are never read, so a page needs no clearing when it is reused.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

PAGE_TOKENS = 64


def pages_for(tokens: int, page_tokens: int = PAGE_TOKENS) -> int:
    return (tokens + page_tokens - 1) // page_tokens


class CacheFullError(RuntimeError):
    """No free page or slot is left: the reference's "context full" (src/model.rs:977-979)."""


class PagePool:
    """Free list of page numbers.  Page 0 is never handed out: padding rows of a fixed-size
    launch write there, so that they change nothing a live sequence reads."""

    TRASH_PAGE = 0

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise ValueError("a pool needs at least one usable page")
        self.n_pages = n_pages            # usable pages, numbered 1..n_pages
        self._free: List[int] = list(range(n_pages, 0, -1))
        self._held = [False] * (n_pages + 1)

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFullError(f"the cache is full: {n} more pages wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if p <= 0 or p > self.n_pages or not self._held[p]:
                raise RuntimeError(f"page {p} is given back but not held")
            self._held[p] = False
            self._free.append(p)


class SlotAllocator:
    """Slot numbers 0..max_slots-1, lowest free number first (so a later batch lands where an
    earlier one was)."""

    def __init__(self, max_slots: int):
        if max_slots < 1:
            raise ValueError("max_slots must be at least 1")
        self.max_slots = max_slots
        self._free = list(range(max_slots - 1, -1, -1))
        self._live = [False] * max_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def live(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and self._live[slot]

    def take(self) -> int:
        if not self._free:
            raise CacheFullError(f"all {self.max_slots} slots are in use")
        # lowest number first
        self._free.sort(reverse=True)
        s = self._free.pop()
        self._live[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not self.live(slot):
            raise RuntimeError(f"slot {slot} is given back but not held")
        self._live[slot] = False
        self._free.append(slot)

    def live_slots(self) -> List[int]:
        return [s for s in range(self.max_slots) if self._live[s]]
