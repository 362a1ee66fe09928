"""Host-side bookkeeping of the cache: which slots and pages are free, and what each
sequence holds.  Pure Python, no device: it can be tested anywhere.

A *slot* is one live sequence.  Each cache *group* (layers with the same needs)
has a pool of pages of ``page_size`` positions; a slot holds, per group, the
list of pages that cover its positions.  The reference has one contiguous
cache for one sequence and zero-fills it per request
(crates/bitnet-core/src/llama/model.rs:29-51, runtime.rs:40); here giving a
slot back is O(pages) and nothing is cleared, because no kernel reads past a
sequence's length.
"""
from __future__ import annotations

from typing import Dict, List


class CacheFull(RuntimeError):
    """No free slot, or no free page, for what was asked."""


class ContextOverflow(RuntimeError):
    """A sequence would grow past the longest length the cache was built for
    (the reference's "sequence position >= max_seq",
    crates/bitnet-core/src/llama/model.rs:221-223)."""


class FreeList:
    """Integers 0..n-1, handed out and taken back; refuses a double give-back."""

    def __init__(self, n: int):
        self.n = n
        self._free = list(range(n - 1, -1, -1))   # pop() hands out low numbers first
        self._held = set()

    def take(self) -> int:
        if not self._free:
            raise CacheFull("none free")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give(self, i: int) -> None:
        if i not in self._held:
            raise ValueError(f"{i} is not held (given back twice, or never taken)")
        self._held.remove(i)
        self._free.append(i)

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def held(self):
        return frozenset(self._held)


class SlotBook:
    """Slots, their lengths and their pages in every group."""

    def __init__(self, n_slots: int, pages_per_group: List[int], page_size: int, max_seq: int):
        self.page_size, self.max_seq = page_size, max_seq
        self.slots = FreeList(n_slots)
        self.pools = [FreeList(n) for n in pages_per_group]
        self.length: Dict[int, int] = {}
        self.pages: Dict[int, List[List[int]]] = {}

    def alloc(self) -> int:
        try:
            s = self.slots.take()
        except CacheFull:
            raise CacheFull(f"all {self.slots.n} slots are in use") from None
        self.length[s] = 0
        self.pages[s] = [[] for _ in self.pools]
        return s

    def free(self, slot: int) -> None:
        if slot not in self.length:
            raise ValueError(f"slot {slot} is not live (freed twice, or never given out)")
        for pool, pages in zip(self.pools, self.pages[slot]):
            for p in pages:
                pool.give(p)
        del self.pages[slot], self.length[slot]
        self.slots.give(slot)

    def reserve(self, slot: int, n_new: int) -> List[List[int]]:
        """Make room for ``n_new`` more positions.  Returns, per group, the pages that
        were added (so the device tables can be brought up to date).  On failure
        nothing is kept."""
        if slot not in self.length:
            raise ValueError(f"slot {slot} is not live")
        total = self.length[slot] + n_new
        if total > self.max_seq:
            raise ContextOverflow(f"sequence would reach {total} positions; the cache holds "
                                  f"at most {self.max_seq} per sequence")
        have = self.pages[slot]
        if all(total <= len(pg) * self.page_size for pg in have):
            return [[] for _ in have]            # the usual case of a decode step: room in the last page
        want = -(-total // self.page_size)
        added = [[] for _ in self.pools]
        try:
            for g, pool in enumerate(self.pools):
                while len(self.pages[slot][g]) + len(added[g]) < want:
                    added[g].append(pool.take())
        except CacheFull:
            for g, pool in enumerate(self.pools):
                for p in added[g]:
                    pool.give(p)
            raise CacheFull(f"no free page for slot {slot}: {total} positions need {want} pages of "
                            f"{self.page_size}") from None
        for g in range(len(self.pools)):
            self.pages[slot][g].extend(added[g])
        return added

    def advance(self, slot: int, n_new: int) -> None:
        new_len = self.length[slot] + n_new
        for pages in self.pages[slot]:
            if new_len > len(pages) * self.page_size:
                raise ValueError(f"slot {slot}: advancing to {new_len} positions, past its reserved pages")
        self.length[slot] = new_len

    def live(self):
        return sorted(self.length)
