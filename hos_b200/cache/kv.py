"""Paged storage of keys and values.

A `KVGroup` serves all entries of the run order whose mixers have the same need
(kv heads, head size, all keys or a window).  It owns a pool of pages of 64
positions, one page table (a row per slot), and for each of its entries a key and
a value array [n_pages, n_kv_heads, 64, head_dim].  A sequence's pages are the
same for every entry of the group: table entry e of a slot names the page that
holds positions 64e..64e+63 (all-keys group) or, in a window group, the positions
p with (p // 64) % ring_pages == e: a ring of ring_pages = ceil(window / 64) pages
that is written round and round.

The host keeps the table and the lengths; `flush()` copies changed rows to the
device before a step runs.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..errors import CacheError
from ..parts.base import KVNeed
from .pool import IdPool

PAGE = ops.PAGE_TOKENS


class KVGroup:
    def __init__(self, need: KVNeed, n_entries: int, n_pages: int, n_slots: int,
                 max_seq_len: int, dtype: torch.dtype, device: torch.device, chunk_tokens: int = 1):
        self.need = need
        self.n_entries = n_entries
        # A step that continues a sequence by n tokens stores all n before any of them attends, so
        # the ring must still hold the window of the first while it holds the last: window + n - 1
        # positions.  `chunk_tokens` is the n the ring is made for (a sequence holds at most
        # ceil(length / 64) pages in any case, so a longer ring costs nothing until it is filled).
        self.ring_pages = 0 if need.window is None else (need.window + max(1, chunk_tokens) - 1 + PAGE - 1) // PAGE
        full_entries = (max_seq_len + PAGE - 1) // PAGE
        self.table_stride = max(1, min(full_entries, self.ring_pages) if self.ring_pages else full_entries)
        self.pages = IdPool(n_pages, "page")
        shape = (n_pages, need.n_kv_heads, PAGE, need.head_dim)
        # zero-filled once: a page's unwritten rows are never selected by a mask, but they
        # are multiplied by zero weights, and 0 * NaN would not be 0
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_entries)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_entries)]
        self.table_host = torch.zeros((n_slots, self.table_stride), dtype=torch.int32)
        self.table_dev = torch.zeros((n_slots, self.table_stride), dtype=torch.int32, device=device)
        self._slot_pages: Dict[int, List[int]] = {}
        self._dirty: set = set()

    def chunk_room(self):
        """The most tokens a sequence may bring in one step that attends over this group's
        storage (None: any number)."""
        if self.ring_pages == 0:
            return None
        return self.ring_pages * PAGE - self.need.window + 1

    def pages_for(self, length: int) -> int:
        n = (length + PAGE - 1) // PAGE
        return min(n, self.table_stride)

    def open_slot(self, slot: int) -> None:
        if slot in self._slot_pages:
            raise CacheError(f"slot {slot} is opened twice")
        self._slot_pages[slot] = []

    def grow(self, slot: int, new_len: int) -> None:
        """Make sure the slot has pages for positions < new_len."""
        held = self._slot_pages[slot]
        want = self.pages_for(new_len)
        if self.ring_pages == 0 and (new_len + PAGE - 1) // PAGE > self.table_stride:
            raise CacheError(f"a sequence of {new_len} tokens is longer than the cache's tables "
                             f"hold ({self.table_stride * PAGE})")
        while len(held) < want:
            page = self.pages.take()
            self.table_host[slot, len(held)] = page
            held.append(page)
            self._dirty.add(slot)

    def close_slot(self, slot: int) -> None:
        for page in self._slot_pages.pop(slot):
            self.pages.give_back(page)

    def flush(self) -> None:
        """Changed rows of the table go to the device: staged in pinned memory (the host may change the
        table again before the copy runs), one asynchronous copy per run of neighbouring rows, no kernel."""
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        on_gpu = self.table_dev.device.type == "cuda"
        staged = torch.empty((len(rows), self.table_stride), dtype=torch.int32, pin_memory=on_gpu)
        torch.index_select(self.table_host, 0, torch.tensor(rows, dtype=torch.long), out=staged)
        at = 0
        while at < len(rows):
            end = at + 1
            while end < len(rows) and rows[end] == rows[end - 1] + 1:
                end += 1
            self.table_dev[rows[at]:rows[at] + end - at].copy_(staged[at:end], non_blocking=on_gpu)
            at = end

    def view(self, entry: int) -> ops.PagedKVArgs:
        return ops.PagedKVArgs(self.k[entry], self.v[entry], self.table_dev, self.ring_pages,
                               self.need.n_kv_heads, self.need.head_dim)

    def bytes_per_token(self) -> int:
        e = self.k[0].element_size()
        return 2 * self.n_entries * self.need.n_kv_heads * self.need.head_dim * e
