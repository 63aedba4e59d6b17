"""Host-side bookkeeping of the cache: which pages and which slots are in use.

Pure Python, no device: the rules that must never break (a page or a slot is never
held twice, never freed twice, never lost) live here and are tested without a GPU.
QStream's arena hands out memory once and resets it as a whole (src/arena.c:67-108);
a batch server needs pieces given back and used again, hence free lists.
"""
from __future__ import annotations

from ..errors import QsError, QStreamError


class PagePool:
    """`n_pages` equal pages; `alloc` hands out the lowest free page number."""

    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise QStreamError(QsError.INVALID_INPUT, f"page pool of {n_pages} pages")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))      # stack; lowest number on top
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise QStreamError(QsError.BUDGET_EXCEEDED,
                               f"the cache's {self.n_pages} pages are all in use")
        page = self._free.pop()
        if self._held[page]:
            raise QStreamError(QsError.INTERNAL, f"page {page} handed out twice")
        self._held[page] = True
        return page

    def free(self, page: int) -> None:
        if not 0 <= page < self.n_pages or not self._held[page]:
            raise QStreamError(QsError.INTERNAL, f"page {page} freed but not held")
        self._held[page] = False
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise QStreamError(QsError.INTERNAL, "a page is twice in the free list")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise QStreamError(QsError.INTERNAL, f"page {p} is {'both held and free' if self._held[p] else 'lost'}")


class SlotTable:
    """One slot per live sequence, with the sequence's length."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise QStreamError(QsError.INVALID_INPUT, f"slot table of {n_slots} slots")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self.active = [False] * n_slots
        self.length = [0] * n_slots
        self.generation = [0] * n_slots          # how often the slot has been handed out

    @property
    def n_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise QStreamError(QsError.BUDGET_EXCEEDED, f"all {self.n_slots} sequence slots are in use")
        s = self._free.pop()
        if self.active[s]:
            raise QStreamError(QsError.INTERNAL, f"slot {s} handed out twice")
        self.active[s] = True
        self.length[s] = 0
        self.generation[s] += 1
        return s

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots or not self.active[slot]:
            raise QStreamError(QsError.INVALID_INPUT, f"slot {slot} released but not held")
        self.active[slot] = False
        self.length[slot] = 0
        self._free.append(slot)

    def require(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots or not self.active[slot]:
            raise QStreamError(QsError.INVALID_INPUT, f"slot {slot} is not held by a sequence")

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise QStreamError(QsError.INTERNAL, "a slot is twice in the free list")
        for s in range(self.n_slots):
            if self.active[s] == (s in free):
                raise QStreamError(QsError.INTERNAL, f"slot {s} is {'both held and free' if self.active[s] else 'lost'}")
