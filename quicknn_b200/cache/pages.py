"""Host-side bookkeeping of the cache: a pool of fixed-size pages and a table of slots.

Both are plain free lists with the invariants that the tests check: nothing is
lost, nothing is held twice, nothing is freed twice.
"""
from __future__ import annotations

from typing import Iterable, List

PAGE = 64          # positions per page of the cache; everything that rounds token counts uses this one

class CacheFull(RuntimeError):
    """The request does not fit: no free page or no free slot.  Raised on the host
    before anything is launched (the reference raises "KV context capacity
    exceeded", src/models/QuickNN.Models.LLM.pas:479-480)."""


class PagePool:
    """Pages 1..n_pages-1 can be handed out; page 0 is never handed out: unused
    page-table entries point at it, so a stray read or a padding row's write lands
    in memory that no sequence owns."""

    def __init__(self, n_pages: int):
        if n_pages < 2:
            raise ValueError("a page pool needs at least one usable page besides page 0")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, 0, -1))   # pop() gives the lowest id first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - 1 - len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} pages wanted, {len(self._free)} free of {self.n_pages - 1}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages: Iterable[int]) -> None:
        for p in pages:
            if p <= 0 or p >= self.n_pages:
                raise ValueError(f"page {p} is not a page of this pool")
            if not self._held[p]:
                raise RuntimeError(f"page {p} is freed twice or was never handed out")
            self._held[p] = False
            self._free.append(p)

    def audit(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(1, self.n_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")
        if self._held[0] or 0 in free:
            raise AssertionError("page 0 left its place")


class SlotTable:
    """Sequence slots 0..n-1; the lowest free id is handed out first, so a slot that
    was given back is used again at once."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise ValueError("at least one slot is needed")
        self.n_slots = n_slots
        self._live = [False] * n_slots

    def take(self) -> int:
        for s, live in enumerate(self._live):
            if not live:
                self._live[s] = True
                return s
        raise CacheFull(f"all {self.n_slots} sequence slots are in use")

    def give_back(self, slot: int) -> None:
        if slot < 0 or slot >= self.n_slots:
            raise ValueError(f"slot {slot} does not exist")
        if not self._live[slot]:
            raise RuntimeError(f"slot {slot} is freed twice or was never handed out")
        self._live[slot] = False

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def live(self) -> List[int]:
        return [s for s, l in enumerate(self._live) if l]

    @property
    def n_free(self) -> int:
        return self._live.count(False)
