"""The cache of a model: a slot per live sequence; for each group of entries with the
same need a paged key/value store of its own; and per-sequence state of fixed size.

Sized by `max_tokens`: the most tokens that live sequences hold at any time, each
sequence's count rounded up to a multiple of 64 (the page size).  Every group gets
max_tokens / 64 pages, which is enough by construction: a sequence of n tokens
holds ceil(n / 64) pages in an all-keys group and at most that many in a window
group.

    slots = cache.admit(lengths)         # one slot per sequence, pages for its prompt
    cache.extend(slot, new_len)          # before a step that lengthens the sequence
    cache.release(slot)                  # the sequence has ended: slot and pages go back

Per-sequence state of fixed size lives beside the keys and values, a row per slot,
zeroed when a sequence is admitted to the slot: the record (`record`, int32
[n_slots, 8]: position, last sampled token, finished flag, count of sampled
tokens, generator state, limit; `recent`, the ring of the tokens sampled last),
which single-token steps read and write on the device (csrc/slot_state.cu), and
whatever a mixer asks for (`StateNeed`: a tensor [n_slots, *shape] per entry and
name; Gemma-2's mixers ask for none).  The host keeps the lengths too (`lengths`),
because it hands out the pages; the kernels of a single-token step take positions
from the record.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import CacheError
from ..parts.base import CallStore, KVNeed, StateNeed
from .kv import KVGroup, PAGE
from .pool import IdPool

RECORD_WORDS, RECENT_TOKENS = 8, 256       # as csrc/slot_state.cu lays a record out
STATE_ONLY_SLOTS = 256                     # slots of a model that keeps no keys, unless max_slots says otherwise


class CacheManager:
    def __init__(self, kv_needs: Sequence[Optional[KVNeed]], cache_from: Sequence[Optional[int]],
                 state_needs: Sequence[Sequence[StateNeed]], max_tokens: int, max_seq_len: int,
                 dtype: torch.dtype, device: torch.device, max_slots: Optional[int] = None,
                 chunk_tokens: int = 1):
        """kv_needs[i], cache_from[i], state_needs[i] describe entry i of the run order.
        `chunk_tokens`: the most tokens one step adds to a sequence that is under way (a window
        group's ring is made long enough for it; longer additions are cut by the step function)."""
        if max_tokens <= 0:
            raise CacheError("the cache must hold at least one token")
        self.device = torch.device(device)
        self.n_pages = (max_tokens + PAGE - 1) // PAGE
        keeps_keys = any(need is not None for need in kv_needs)
        # What bounds a sequence and the number of slots: the pages, where keys and values are kept (a sequence
        # cannot be longer than all pages hold, and every live sequence holds a page at least); a model whose
        # mixers keep state of fixed size only is bounded by neither, so its slots are simply counted.
        self.max_seq_len = min(max_seq_len, self.n_pages * PAGE) if keeps_keys else max_seq_len
        self.n_slots = max(1, min(self.n_pages, max_slots or 4096)) if keeps_keys else max(1, max_slots or STATE_ONLY_SLOTS)
        self.slots = IdPool(self.n_slots, "slot")
        self.lengths: Dict[int, int] = {}
        # group entries by need
        self.groups: List[KVGroup] = []
        self._entry_group: List[Optional[Tuple[int, int]]] = []     # entry -> (group, index in group)
        by_need: Dict[KVNeed, List[int]] = {}
        for i, need in enumerate(kv_needs):
            if need is not None and cache_from[i] is None:
                by_need.setdefault(need, []).append(i)
        placed: Dict[int, Tuple[int, int]] = {}
        for need, entries in by_need.items():
            g = KVGroup(need, len(entries), self.n_pages, self.n_slots, self.max_seq_len, dtype,
                        self.device, chunk_tokens)
            for j, e in enumerate(entries):
                placed[e] = (len(self.groups), j)
            self.groups.append(g)
        self.stores: List[CallStore] = []
        for i, need in enumerate(kv_needs):
            src = cache_from[i]
            kv, owns = None, True
            if need is not None:
                owner = i if src is None else src
                if owner not in placed:
                    raise CacheError(f"entry {i} reads the cache of entry {src}, which keeps none")
                gi, j = placed[owner]
                if src is not None and kv_needs[src] != need:
                    raise CacheError(f"entry {i} reads the cache of entry {src}, whose keys have "
                                     f"another shape or window")
                kv, owns = self.groups[gi].view(j), src is None
            state = {s.name: torch.zeros((self.n_slots,) + tuple(s.shape), dtype=s.dtype,
                                         device=self.device) for s in state_needs[i]}
            self.stores.append(CallStore(kv, owns, state))
        self.record = torch.zeros((self.n_slots, RECORD_WORDS), dtype=torch.int32, device=self.device)
        self.recent = torch.zeros((self.n_slots, RECENT_TOKENS), dtype=torch.int32, device=self.device)

    # ---- sequences ------------------------------------------------------------------
    def admit(self, lengths: Sequence[int]) -> List[int]:
        """Slots for new sequences whose first step brings `lengths` tokens.  All or nothing."""
        need_pages = [sum(g.pages_for(n) for n in lengths) for g in self.groups]
        for g, want in zip(self.groups, need_pages):
            if want > g.pages.n_free:
                raise CacheError(f"the cache cannot hold these sequences: {want} pages wanted, "
                                 f"{g.pages.n_free} free of {g.pages.n}")
        if len(lengths) > self.slots.n_free:
            raise CacheError(f"the cache has {self.slots.n_free} free slots, {len(lengths)} wanted")
        for n in lengths:
            if n > self.max_seq_len:
                raise CacheError(f"a sequence of {n} tokens is longer than the cache holds "
                                 f"({self.max_seq_len})")
        out = []
        for n in lengths:
            slot = self.slots.take()
            self.lengths[slot] = 0
            for g in self.groups:
                g.open_slot(slot)
            out.append(slot)
        at = 0
        ordered = sorted(out)
        while at < len(ordered):                       # runs of neighbouring slots are cleared together
            end = at + 1
            while end < len(ordered) and ordered[end] == ordered[end - 1] + 1:
                end += 1
            lo, hi = ordered[at], ordered[end - 1] + 1
            self.record[lo:hi].zero_()
            for st in self.stores:
                for t in st.state.values():
                    t[lo:hi].zero_()
            at = end
        return out

    def extend(self, slot: int, new_len: int) -> None:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} holds no sequence")
        if new_len > self.max_seq_len:
            raise CacheError(f"a sequence of {new_len} tokens is longer than the cache holds "
                             f"({self.max_seq_len})")
        for g in self.groups:          # all or nothing: look before taking
            more = g.pages_for(new_len) - len(g._slot_pages[slot])
            if more > g.pages.n_free:
                raise CacheError(f"the cache has no free page left for slot {slot} to reach "
                                 f"{new_len} tokens ({more} wanted, {g.pages.n_free} free)")
        for g in self.groups:
            g.grow(slot, new_len)
        self.lengths[slot] = max(self.lengths[slot], new_len)

    def extend_all(self, slots: Sequence[int], new_lens: Sequence[int]) -> None:
        """`extend` for the sequences of one step, all or nothing: if any of them cannot have
        its pages (or would pass the longest sequence the cache holds), none is changed."""
        for slot, n in zip(slots, new_lens):
            if slot not in self.lengths:
                raise CacheError(f"slot {slot} holds no sequence")
            if n > self.max_seq_len:
                raise CacheError(f"a sequence of {n} tokens is longer than the cache holds "
                                 f"({self.max_seq_len})")
        for g in self.groups:
            more = sum(max(0, g.pages_for(n) - len(g._slot_pages[slot])) for slot, n in zip(slots, new_lens))
            if more > g.pages.n_free:
                raise CacheError(f"the cache has no free pages left for this step ({more} wanted, "
                                 f"{g.pages.n_free} free of {g.pages.n})")
        for slot, n in zip(slots, new_lens):
            for g in self.groups:
                g.grow(slot, n)
            self.lengths[slot] = max(self.lengths[slot], n)

    def chunk_room(self) -> Optional[int]:
        """The most tokens one step may add to a sequence that is under way (None: any number):
        the smallest room of the window groups' rings."""
        rooms = [r for r in (g.chunk_room() for g in self.groups) if r is not None]
        return min(rooms) if rooms else None

    def release(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is released but holds no sequence (freed twice?)")
        for g in self.groups:
            g.close_slot(slot)
        del self.lengths[slot]
        self.slots.give_back(slot)

    def flush(self) -> None:
        for g in self.groups:
            g.flush()

    def check(self) -> None:
        """No slot or page lost, held twice or freed twice."""
        self.slots.check()
        if self.slots.held() != set(self.lengths):
            raise CacheError("held slots and live sequences differ")
        for g in self.groups:
            g.pages.check()
            owned = [p for pages in g._slot_pages.values() for p in pages]
            if len(owned) != len(set(owned)):
                raise CacheError("a page is held by two sequences")
            if set(owned) != g.pages.held():
                raise CacheError("held pages and the sequences' pages differ")

    def tokens_capacity(self) -> int:
        """Tokens the live sequences may hold in all (each rounded up to `page_tokens`); without keys and values
        to keep, no bound."""
        return self.n_pages * PAGE if self.groups else 1 << 62

    @property
    def page_tokens(self) -> int:
        """The unit in which a sequence takes room (1 where nothing grows with a sequence's length)."""
        return PAGE if self.groups else 1

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)
