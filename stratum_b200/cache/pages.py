"""Host-side bookkeeping of the cache: sequence slots and pages of key/value rows.

The reference gives every stream of a batch one slot of a fixed capacity
(stratum/native/stratum_arch_llama.inc.c:271-285, :1458-1470) and treats
overflow as an error, never a wrap (:689-695).  Here a slot owns a list of
pages (PAGE_TOKENS rows each) taken from a shared pool, so capacity is counted
in tokens held by live sequences, whatever their mix of lengths; a released
slot hands its pages back and both are used again.  All of this is plain
Python and is tested without a GPU.
"""
from __future__ import annotations

from typing import Dict, List, Optional

PAGE_TOKENS = 64


class CacheFull(RuntimeError):
    """No free slot, or fewer free pages than the step needs."""


class CacheMisuse(RuntimeError):
    """A slot or page was released twice, or used without being held."""


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


class PagePool:
    """Free list of page numbers 0..n_pages-1.  Lowest numbers are handed out first."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))   # pop() yields the lowest
        self._held = [False] * n_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"cache needs {n} more pages of {PAGE_TOKENS} tokens, {len(self._free)} are free "
                            f"(of {self.n_pages})")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give(self, pages: List[int]) -> None:
        seen = set()
        for p in pages:                       # check everything first: a refused give changes nothing
            if not (0 <= p < self.n_pages) or not self._held[p] or p in seen:
                raise CacheMisuse(f"page {p} given back but not held")
            seen.add(p)
        for p in pages:
            self._held[p] = False
        # keep the free list sorted descending so that take() stays lowest-first and deterministic
        self._free.extend(pages)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every page is either free or held, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheMisuse("a page is on the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise CacheMisuse(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")


class SlotTable:
    """Sequence slots 0..max_slots-1; the lowest free one is handed out first."""

    def __init__(self, max_slots: int):
        if max_slots < 1:
            raise ValueError("a slot table needs at least one slot")
        self.max_slots = max_slots
        self._free: List[int] = list(range(max_slots - 1, -1, -1))
        self._live = [False] * max_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def live(self) -> List[int]:
        return [s for s in range(self.max_slots) if self._live[s]]

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and self._live[slot]

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.max_slots} sequence slots are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def release(self, slot: int) -> None:
        if not self.is_live(slot):
            raise CacheMisuse(f"slot {slot} released but not held")
        self._live[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheMisuse("a slot is on the free list twice")
        for s in range(self.max_slots):
            if self._live[s] == (s in free):
                raise CacheMisuse(f"slot {s} is {'both live and free' if self._live[s] else 'lost'}")


class SequencePages:
    """The pages one sequence holds in one group of layers.

    `window` = 0 keeps every key; `window` = W keeps only what the next query can
    still see (the last W positions), so pages that fall wholly behind the window
    go back to the pool as the sequence grows.  Entry i of `table` is the page
    that holds positions [i*PAGE_TOKENS, (i+1)*PAGE_TOKENS), or -1 once dropped.
    """

    def __init__(self, pool: PagePool, window: int = 0):
        self.pool = pool
        self.window = window
        self.table: List[int] = []
        self.length = 0

    def pages_needed(self, n_new: int) -> int:
        return max(0, pages_for(self.length + n_new) - len(self.table))

    def reserve(self, n_new: int) -> None:
        self.table.extend(self.pool.take(self.pages_needed(n_new)))

    def advance(self, n_new: int) -> bool:
        """The sequence now holds n_new more positions.  True if that changed the page table (a windowed
        group handed pages back)."""
        self.length += n_new
        if self.length > len(self.table) * PAGE_TOKENS:
            raise CacheMisuse("sequence advanced beyond its reserved pages")
        if self.window > 0:
            first_needed = max(0, self.length - self.window + 1) // PAGE_TOKENS
            drop = [p for p in self.table[:first_needed] if p >= 0]
            if drop:
                self.pool.give(drop)
                for i in range(first_needed):
                    self.table[i] = -1
                return True
        return False

    def release(self) -> None:
        self.pool.give([p for p in self.table if p >= 0])
        self.table = []
        self.length = 0
