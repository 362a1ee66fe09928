"""Host-side bookkeeping of the cache: which slots and pages are free, and what each
sequence holds.  Pure Python, no device: it can be tested anywhere.

A *slot* is one live sequence.  Each cache *group* (layers with the same needs)
has a pool of pages of ``page_size`` positions; a slot holds, per group, the
list of pages that cover its positions.  The reference has one contiguous
cache for one sequence and zero-fills it per request
(crates/bitnet-core/src/llama/model.rs:29-51, runtime.rs:40); here giving a
slot back is O(pages) and nothing is cleared, because no kernel reads past a
sequence's length.

A group whose layers see only the last ``window`` keys gives a sequence's pages
back as soon as they lie wholly behind the window of the sequence's next token
(the attention kernels start at the page that holds the first visible key), so
a long sequence holds about ``window / page_size + 2`` pages of such a group,
whatever its length.  The released places of a page list hold -1.
"""
from __future__ import annotations

from typing import Dict, List, Optional


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

    def __init__(self, n_slots: int, pages_per_group: List[int], page_size: int, max_seq: int,
                 windows: Optional[List[Optional[int]]] = None):
        self.page_size, self.max_seq = page_size, max_seq
        self.slots = FreeList(n_slots)
        self.pools = [FreeList(n) for n in pages_per_group]
        #: per group, how many of the last keys its layers see (None: all of them)
        self.windows = list(windows) if windows is not None else [None] * len(pages_per_group)
        self.has_windows = any(w for w in self.windows)
        self.length: Dict[int, int] = {}
        self.pages: Dict[int, List[List[int]]] = {}
        self._released: Dict[int, List[int]] = {}      # per slot and group: leading pages given back

    def alloc(self) -> int:
        try:
            s = self.slots.take()
        except CacheFull:
            raise CacheFull(f"all {self.slots.n} slots are in use") from None
        self.length[s] = 0
        self.pages[s] = [[] for _ in self.pools]
        self._released[s] = [0] * len(self.pools)
        return s

    def free(self, slot: int) -> None:
        if slot not in self.length:
            raise ValueError(f"slot {slot} is not live (freed twice, or never given out)")
        for pool, pages in zip(self.pools, self.pages[slot]):
            for p in pages:
                if p >= 0:
                    pool.give(p)
        del self.pages[slot], self.length[slot], self._released[slot]
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
        if self.has_windows:
            self.release_behind_window(slot)

    def release_behind_window(self, slot: int) -> None:
        """Gives back the pages of windowed groups that no later token of the sequence can see: the
        next token sits at position ``length`` and sees keys from ``length - window + 1`` on."""
        n = self.length[slot]
        for g, w in enumerate(self.windows):
            if not w:
                continue
            pages = self.pages[slot][g]
            first_needed = min(max(0, n - w + 1) // self.page_size, len(pages))
            for i in range(self._released[slot][g], first_needed):
                self.pools[g].give(pages[i])
                pages[i] = -1
            if first_needed > self._released[slot][g]:
                self._released[slot][g] = first_needed

    def pages_needed(self, group: int, prompt: int, grown: int) -> int:
        """Most pages of ``group`` that a sequence holds at any time if its prompt of ``prompt`` tokens
        runs in one step and it then grows token by token to ``grown`` positions."""
        whole = -(-int(grown) // self.page_size)
        w = self.windows[group]
        if not w:
            return whole
        return min(whole, max(-(-int(prompt) // self.page_size), (w - 1) // self.page_size + 2))

    def live(self):
        return sorted(self.length)
