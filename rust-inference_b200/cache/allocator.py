"""Host-side bookkeeping of the cache: which slots are live, which pages each
slot maps, how long each sequence is.  No device memory is touched here.

The paged design is thanhauco/rust-inference's (src/kvcache.rs:12-61,
106-135): fixed pages of ``page_size`` tokens, a page table row per sequence
with -1 for "unmapped", pages handed out from a free list as a sequence grows
(lowest page first).  Added to it: a row is a *slot* that is given out and
taken back per sequence, sequences grow by different amounts in one step, and
a slot's pages return to the free list when the slot is freed.
"""
from __future__ import annotations

from typing import List

import numpy as np


class CacheError(RuntimeError):
    """Out of slots or pages, a sequence over its limit, or a misuse of a slot."""


class SlotAllocator:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise CacheError("the cache needs at least one slot")
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots - 1, -1, -1))   # pop() gives slot 0 first
        self._live = [False] * num_slots

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.num_slots} cache slots are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def free(self, slot: int) -> None:
        self.require_live(slot)
        self._live[slot] = False
        self._free.append(slot)

    def require_live(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots) or not self._live[slot]:
            raise CacheError(f"slot {slot} is not live")

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.num_slots and self._live[slot]

    @property
    def live_count(self) -> int:
        return self.num_slots - len(self._free)

    def check(self) -> None:
        """Every slot is either free or live, never both, never twice."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise AssertionError("a slot is in the free list twice")
        live = [s for s in range(self.num_slots) if self._live[s]]
        if set(free) & set(live):
            raise AssertionError("a slot is both free and live")
        if len(free) + len(live) != self.num_slots:
            raise AssertionError("a slot was lost")


class PageTable:
    """Pages of one cache group: free list, the table [slots, max_pages_per_seq]
    and the number of tokens stored per slot.

    ``window`` > 0: only the last ``window`` keys are ever read again, so pages
    that lie wholly before them are released after every step.
    """

    def __init__(self, num_slots: int, num_pages: int, max_pages_per_seq: int, page_size: int, window: int = 0):
        if num_pages <= 0 or max_pages_per_seq <= 0 or page_size <= 0:
            raise CacheError("page counts and the page size must be positive")
        self.num_slots, self.num_pages = num_slots, num_pages
        self.max_pages_per_seq, self.page_size, self.window = max_pages_per_seq, page_size, window
        self.table = np.full((num_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.lens = [0] * num_slots
        self._first_mapped = [0] * num_slots        # logical pages below it were released (window)
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives page 0 first
        self.dirty = set()                           # slots whose row changed since the last upload

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def max_seq_len(self) -> int:
        return self.max_pages_per_seq * self.page_size

    def pages_needed(self, slot: int, new_tokens: int) -> int:
        """Pages that ``extend(slot, new_tokens)`` would take from the free list."""
        start, end = self.lens[slot], self.lens[slot] + new_tokens
        row = self.table[slot]
        last = min(-(-end // self.page_size), self.max_pages_per_seq)
        return sum(1 for p in range(start // self.page_size, last) if row[p] < 0)

    def extend(self, slot: int, new_tokens: int) -> int:
        """Map pages for the next ``new_tokens`` positions of ``slot`` and advance
        its length; returns the length before.  Nothing changes if it fails."""
        if new_tokens < 0:
            raise CacheError("a sequence cannot shrink")
        start = self.lens[slot]
        end = start + new_tokens
        if end > self.max_seq_len:
            raise CacheError(f"slot {slot} would reach {end} tokens, the cache holds {self.max_seq_len} per sequence")
        row = self.table[slot]
        need = [p for p in range(start // self.page_size, -(-end // self.page_size)) if row[p] < 0]
        if len(need) > len(self._free):
            raise CacheError(f"cache out of pages: {len(need)} needed, {len(self._free)} of {self.num_pages} free")
        for p in need:
            row[p] = self._free.pop()
        if need:
            self.dirty.add(slot)
        self.lens[slot] = end
        return start

    def release_behind_window(self, slot: int) -> int:
        """Give back the pages that no later query of ``slot`` can see (window groups)."""
        if self.window <= 0:
            return 0
        first_needed = self.lens[slot] - self.window + 1      # oldest key the next query reads
        row, n = self.table[slot], 0
        p = self._first_mapped[slot]
        while (p + 1) * self.page_size <= first_needed:
            if row[p] >= 0:
                self._free.append(int(row[p]))
                row[p] = -1
                n += 1
            p += 1
        self._first_mapped[slot] = p
        if n:
            self.dirty.add(slot)
        return n

    def release(self, slot: int) -> None:
        """Give back every page of ``slot`` and reset its length."""
        row = self.table[slot]
        mapped = row[row >= 0]
        self._free.extend(int(p) for p in mapped[::-1])
        if len(mapped):
            row[:] = -1
            self.dirty.add(slot)
        self.lens[slot] = 0
        self._first_mapped[slot] = 0

    def check(self) -> None:
        """Every page is free or mapped exactly once."""
        mapped = self.table[self.table >= 0].tolist()
        if len(set(mapped)) != len(mapped):
            raise AssertionError("a page is mapped twice")
        if len(set(self._free)) != len(self._free):
            raise AssertionError("a page is in the free list twice")
        if set(mapped) & set(self._free):
            raise AssertionError("a page is both free and mapped")
        if len(mapped) + len(self._free) != self.num_pages:
            raise AssertionError("a page was lost")
