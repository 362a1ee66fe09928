"""Device storage of the cache: pages of keys and values per group of layers, page
tables, and the fixed-size per-sequence state area.

Layout of one group: per stored tensor ("stream": keys and values by default, whatever a
mixer's ``CacheNeed.streams`` names otherwise) a pool
``[layer in group][page][head][position in page][width]`` in the engine's compute dtype.
A head's page is one contiguous [page_size, width] tile.  ``table[slot][i]`` is the page
that holds the slot's positions i*page_size .. (i+1)*page_size-1; the streams of a group
share the table.

State area: for every schedule entry whose mixer declares a ``StateNeed``, a
tensor [n_slots, *shape]; a slot's rows are zeroed when the slot is given out.
The Llama decoder needs none, so the area is empty for it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..parts.base import CacheNeed, StateNeed
from .allocator import SlotBook, CacheFull, ContextOverflow  # noqa: F401

PAGE_SIZE = 64


@dataclass
class CacheLayerView:
    """What a mixer sees of the cache for one run of a layer."""
    k: torch.Tensor            # [n_pages, kv heads, page_size, head_dim]: the first stream
    v: Optional[torch.Tensor]  # the second stream (None for a group that stores one tensor per position)
    page_table: torch.Tensor   # int32 [n_slots, max_pages], on the device
    max_pages: int
    page_size: int
    n_kv_heads: int
    head_dim: int
    writes: bool               # False: this run reads what another run wrote
    group: int
    streams: tuple = ()        # every stored tensor of this layer, in the order of the need's streams


class CacheGroup:
    def __init__(self, need: CacheNeed, entries: List[int], n_pages: int, n_slots: int, max_pages: int,
                 page_size: int, dtype, device):
        self.need, self.entries = need, entries
        self.n_pages = n_pages
        self.pools = [torch.zeros((len(entries), n_pages, heads, page_size, width), dtype=dtype, device=device)
                      for heads, width in need.stream_shapes()]
        self.table_host = np.zeros((n_slots, max_pages), dtype=np.int32)
        self.table = torch.zeros((n_slots, max_pages), dtype=torch.int32, device=device)
        self.dirty = set()

    def bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools)

    def bytes_per_position(self) -> int:
        """What one cached position of one sequence holds in this group, over its layers."""
        return sum(h * w for h, w in self.need.stream_shapes()) * self.pools[0].element_size() * len(self.entries)


class SequenceCache:
    """Slots for sequences; keys and values for each cached run of a layer; per-sequence state."""

    def __init__(self, cache_needs: Dict[int, CacheNeed], reads: Dict[int, int],
                 state_needs: Dict[int, StateNeed], max_tokens: int, max_seq: int, dtype, device,
                 page_size: int = PAGE_SIZE, n_slots: Optional[int] = None):
        """cache_needs: schedule entry -> need, for entries that write their own keys and values.
        reads: schedule entry -> the entry whose cache it reads.  max_tokens: the most positions
        all live sequences hold together, each rounded up to whole pages."""
        self.page_size = page_size
        self.max_seq = max_seq
        self.max_pages = -(-max_seq // page_size)
        n_pages = max(1, -(-max_tokens // page_size))
        self.n_slots = n_slots if n_slots is not None else n_pages
        self.device, self.dtype = device, dtype
        by_need: Dict[CacheNeed, List[int]] = {}
        for entry in sorted(cache_needs):
            by_need.setdefault(cache_needs[entry], []).append(entry)
        self.groups: List[CacheGroup] = [
            CacheGroup(need, entries, n_pages, self.n_slots, self.max_pages, page_size, dtype, device)
            for need, entries in by_need.items()]
        self._where: Dict[int, tuple] = {}
        for g, grp in enumerate(self.groups):
            for i, entry in enumerate(grp.entries):
                self._where[entry] = (g, i, True)
        for entry, src in reads.items():
            if src not in self._where or not self._where[src][2]:
                raise ValueError(f"schedule entry {entry} reads the cache of entry {src}, which writes none")
            g, i, _ = self._where[src]
            self._where[entry] = (g, i, False)
        self.book = SlotBook(self.n_slots, [grp.n_pages for grp in self.groups], page_size, max_seq,
                             windows=[grp.need.window for grp in self.groups])
        self.states: Dict[int, torch.Tensor] = {
            entry: torch.zeros((self.n_slots, *need.shape), dtype=need.dtype, device=device)
            for entry, need in state_needs.items()}

    # ---- slots
    def alloc(self) -> int:
        slot = self.book.alloc()
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        self.book.free(slot)

    def length(self, slot: int) -> int:
        return self.book.length[slot]

    def reserve(self, slot: int, n_new: int) -> None:
        added = self.book.reserve(slot, n_new)
        for g, pages in enumerate(added):
            if pages:
                have = len(self.book.pages[slot][g])
                self.groups[g].table_host[slot, have - len(pages):have] = pages
                self.groups[g].dirty.add(slot)

    def advance(self, slot: int, n_new: int) -> None:
        self.book.advance(slot, n_new)

    def lengths(self, slots) -> list:
        length = self.book.length
        return [length[s] for s in slots]

    def reserve_one_each(self, slots) -> None:
        """Room for one more position in each slot: the decode step's call, which finds room in the
        last page nearly always and then touches nothing."""
        book = self.book
        page, pages, length, most = book.page_size, book.pages, book.length, book.max_seq
        for s in slots:
            want = length[s] + 1
            if want > most:
                self.reserve(s, 1)           # raises ContextOverflow
                continue
            for pg in pages[s]:
                if want > len(pg) * page:
                    self.reserve(s, 1)
                    break

    def advance_one_each(self, slots) -> None:
        """After ``reserve_one_each``: every slot holds one position more."""
        length = self.book.length
        for s in slots:
            length[s] += 1
        if self.book.has_windows:
            for s in slots:
                self.book.release_behind_window(s)

    def fits(self, lengths, prompts=None) -> bool:
        """Whether new sequences that grow to these lengths fit beside what is live now.  With
        ``prompts`` (the part of each length that arrives in the first step) a windowed group is
        counted by what it holds at most, not by the whole length."""
        if len(lengths) > self.book.slots.n_free:
            return False
        if prompts is None:
            prompts = lengths
        for g, pool in enumerate(self.book.pools):
            if sum(self.book.pages_needed(g, p, n) for p, n in zip(prompts, lengths)) > pool.n_free:
                return False
        return True

    def upload_tables(self) -> None:
        """Bring the device page tables up to date (rows that changed since the last call)."""
        for g, grp in enumerate(self.groups):
            for slot in sorted(grp.dirty):
                n = len(self.book.pages[slot][g]) if slot in self.book.pages else 0
                if n:
                    # a pageable copy: staged by the driver before it returns, so the
                    # host row may change again at once.  (Entries of pages that were given back
                    # behind a window keep their old number: no kernel reads that far back.)
                    grp.table[slot, :n].copy_(torch.from_numpy(grp.table_host[slot, :n].copy()))
            grp.dirty.clear()

    # ---- views
    def view(self, entry: int) -> CacheLayerView:
        g, i, writes = self._where[entry]
        grp = self.groups[g]
        streams = tuple(p[i] for p in grp.pools)
        return CacheLayerView(streams[0], streams[1] if len(streams) > 1 else None, grp.table, self.max_pages,
                              self.page_size, grp.need.n_kv_heads, grp.need.head_dim, writes, g, streams)

    def state(self, entry: int) -> Optional[torch.Tensor]:
        return self.states.get(entry)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + sum(s.numel() * s.element_size()
                                                          for s in self.states.values())
