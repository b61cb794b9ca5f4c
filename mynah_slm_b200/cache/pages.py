"""Host-side bookkeeping of the cache: pages, slots, and what each sequence holds.

A page holds 64 positions of one storage group. A sequence has a slot (its
row in every per-sequence table) and, in every group, the list of pages that
hold its positions. Pages are handed out when a sequence grows into them and
given back when the sequence ends, or, in a group that keeps only a window,
as soon as every position of the page has left the window. Freed pages and
slots are the next to be handed out again, so reuse happens at once.

Nothing here touches the device; the engine turns the lists into the tables
the kernels read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

PAGE_TOKENS = 64


class CacheError(RuntimeError):
    pass


class PagePool:
    """Pages 0..n-1 of one group. Tracks the owner of each page so that a
    page can be neither handed out twice nor given back twice."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))      # stack: page 0 first
        self._owner: list[Optional[int]] = [None] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, n: int, owner: int) -> list[int]:
        if n > len(self._free):
            raise CacheError(f"the cache is full: {n} pages wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._owner[p] is not None:
                raise CacheError(f"page {p} was free and owned by slot {self._owner[p]} at once")
            self._owner[p] = owner
        return out

    def give_back(self, pages: list[int], owner: int) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise CacheError(f"page {p} does not exist")
            if self._owner[p] != owner:
                raise CacheError(f"slot {owner} gives back page {p}, which "
                                 f"{'is free' if self._owner[p] is None else f'belongs to slot {self._owner[p]}'}")
            self._owner[p] = None
            self._free.append(p)

    def owner(self, page: int) -> Optional[int]:
        return self._owner[page]


class SlotTable:
    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise CacheError(f"a slot table needs at least one slot, got {n_slots}")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._used: set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.n_slots} sequence slots are in use")
        s = self._free.pop()
        self._used.add(s)
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._used:
            raise CacheError(f"slot {slot} is not in use")
        self._used.remove(slot)
        self._free.append(slot)

    def in_use(self, slot: int) -> bool:
        return slot in self._used


@dataclass
class GroupPlan:
    """Storage group: the cache entries (runs of layers) that need the same
    thing per position and may therefore share page lists."""
    kv_heads: int
    head_dim: int
    window: Optional[int]          # None: every position is kept
    entries: list[int] = field(default_factory=list)    # schedule indices stored here


@dataclass
class _Held:
    pages: list[int] = field(default_factory=list)
    base: int = 0                  # logical index of pages[0]


class SequencePages:
    """What the live sequences hold, in every group."""

    def __init__(self, groups: list[GroupPlan], n_pages: int, max_seqs: int):
        self.groups = groups
        self.pools = [PagePool(n_pages) for _ in groups]
        self.slots = SlotTable(max_seqs)
        self.length: dict[int, int] = {}
        self._held: dict[int, list[_Held]] = {}

    # ---------------------------------------------------------- lifecycle
    def open(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        self._held[slot] = [_Held() for _ in self.groups]
        return slot

    def close(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open")
        for pool, held in zip(self.pools, self._held[slot]):
            pool.give_back(held.pages, slot)
        del self._held[slot], self.length[slot]
        self.slots.give_back(slot)

    # -------------------------------------------------------------- growth
    def pages_needed(self, slot: int, n_new: int) -> int:
        """Pages the fullest group still has to take for n_new more positions."""
        need_total = -(-(self.length[slot] + n_new) // PAGE_TOKENS)
        return max((need_total - (h.base + len(h.pages)) for h in self._held[slot]), default=0)

    def reserve(self, slot: int, n_new: int) -> None:
        """Make sure every position below length + n_new has a page in every group."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open")
        if n_new < 0:
            raise CacheError("cannot reserve a negative number of positions")
        need_total = -(-(self.length[slot] + n_new) // PAGE_TOKENS)
        wants = [max(0, need_total - (h.base + len(h.pages))) for h in self._held[slot]]
        for pool, w in zip(self.pools, wants):      # all or nothing
            if w > pool.n_free:
                raise CacheError(f"the cache is full: {w} pages wanted, {pool.n_free} of {pool.n_pages} free")
        for pool, held, w in zip(self.pools, self._held[slot], wants):
            held.pages += pool.take(w, slot)

    def commit(self, slot: int, n_new: int) -> None:
        """The positions have been written: advance, and let windowed groups
        give back the pages no later query can see."""
        n = self.length[slot] + n_new
        for g, pool, held in zip(self.groups, self.pools, self._held[slot]):
            if (held.base + len(held.pages)) * PAGE_TOKENS < n:
                raise CacheError(f"slot {slot} advanced to {n} positions without pages for them")
            if g.window is not None:
                first_needed = max(0, n - g.window + 1) // PAGE_TOKENS
                drop = min(first_needed - held.base, len(held.pages))
                if drop > 0:
                    pool.give_back(held.pages[:drop], slot)
                    del held.pages[:drop]
                    held.base += drop
        self.length[slot] = n

    # --------------------------------------------------------------- views
    def held(self, slot: int, group: int) -> tuple[list[int], int]:
        h = self._held[slot][group]
        return h.pages, h.base

    def live_slots(self) -> list[int]:
        return sorted(self.length)
