"""Host-side bookkeeping of the cache: which slots and pages are free, and who holds what.

Nothing here touches a device; the invariants (no slot or page lost, held twice or freed
twice) are checked on every call and tested on the CPU.

The reference has one implicit sequence per model: `KvStorage` keeps a single index of the
tokens stored (`m_store_id`, src/core/kvstorage.h:40-49) in one growable tensor per layer
(src/core/kvstotage.cpp:53-76), and `reset_id` rewinds it (src/core/kvstorage.h:43-46).
Here a sequence holds a slot, and per group of layers a list of fixed-size pages that grows
with its length; both go back to their pools when the sequence ends and are handed to the
next one.
"""
from __future__ import annotations

from typing import Dict, List


class CacheError(RuntimeError):
    """Misuse of the cache: a slot that is not live, a page freed twice, and the like."""


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the step."""


class IndexPool:
    """A pool of the integers 0..n-1.  Lowest index first, so that reuse is deterministic."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))  # pop() gives the lowest
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def alloc(self, count: int = 1) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            if self._held[i]:
                raise CacheError(f"{self.what} {i} was on the free list while held")
            self._held[i] = True
        return out

    def free(self, items) -> None:
        for i in items:
            if not 0 <= i < self.n:
                raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} freed twice (or never handed out)")
            self._held[i] = False
            self._free.append(i)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """Every index is either free exactly once or held."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in range(self.n):
            if self._held[i] == (i in seen):
                raise CacheError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")


class PageLedger:
    """The pages of one group of layers: a pool and, per slot, the pages it holds by logical
    page number.  A windowed group gives pages back once every position in them has left the
    window of all future queries; their logical entry then reads -1."""

    def __init__(self, num_pages: int, page_size: int, num_slots: int, window=None):
        self.pool = IndexPool(num_pages, "page")
        self.page_size = int(page_size)
        self.window = window
        self.pages: List[Dict[int, int]] = [dict() for _ in range(num_slots)]
        self.n_logical = [0] * num_slots  # logical pages ever reserved by the slot's sequence

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, -(-new_len // self.page_size) - self.n_logical[slot])

    def reserve(self, slot: int, new_len: int) -> None:
        """Make sure the slot has pages for positions 0..new_len-1 (those not yet released)."""
        want = -(-new_len // self.page_size)
        first = self.n_logical[slot]
        if want > first:
            for lp, pp in zip(range(first, want), self.pool.alloc(want - first)):
                self.pages[slot][lp] = pp
            self.n_logical[slot] = want

    def release_outside_window(self, slot: int, seq_len: int) -> None:
        """After a step: pages whose positions are all older than the next query's window."""
        if self.window is None:
            return []
        first_needed_pos = seq_len - self.window + 1  # oldest key the next token may see
        if first_needed_pos <= 0:
            return []
        first_page = first_needed_pos // self.page_size
        have = self.pages[slot]
        gone = [have.pop(lp) for lp in [lp for lp in have if lp < first_page]]
        self.pool.free(gone)
        return gone

    def release_all(self, slot: int) -> None:
        have = self.pages[slot]
        gone = list(have.values())
        self.pool.free(gone)
        have.clear()
        self.n_logical[slot] = 0
        return gone

    def row(self, slot: int, width: int, out) -> None:
        """Write the slot's logical->physical table into out[0:width] (-1 = no page)."""
        out[:width] = -1
        for lp, pp in self.pages[slot].items():
            if lp < width:
                out[lp] = pp

    def check(self) -> None:
        self.pool.check()
        held = [p for d in self.pages for p in d.values()]
        if len(held) != len(set(held)):
            raise CacheError("a page is held by two sequences")
        if len(held) != self.pool.n_held:
            raise CacheError(f"{self.pool.n_held} pages are out of the pool but sequences hold {len(held)}")
