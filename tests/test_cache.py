"""The cache's bookkeeping on the host (no GPU): no slot or page lost, held twice or
freed twice; groups with storage of their own; rings; reuse."""
import random

import pytest
import torch

from hos_b200.cache import CacheManager, IdPool
from hos_b200.errors import CacheError
from hos_b200.parts.base import KVNeed, StateNeed

CPU = torch.device("cpu")


def make(max_tokens=1024, window=100, max_seq_len=512, entries=4, **kw):
    # entries alternate: window, all keys, window, all keys ...
    needs = [KVNeed(2, 16, window if i % 2 == 0 else None) for i in range(entries)]
    return CacheManager(needs, [None] * entries, [[] for _ in needs], max_tokens, max_seq_len,
                        torch.float32, CPU, **kw)


def test_id_pool_invariants():
    p = IdPool(3, "slot")
    a, b, c = p.take(), p.take(), p.take()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(CacheError, match="no free slot"):
        p.take()
    p.give_back(b)
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back(b)
    with pytest.raises(CacheError, match="does not exist"):
        p.give_back(7)
    assert p.take() == 1              # the freed id is used again at once
    p.check()


def test_groups_have_storage_of_their_own():
    c = make()
    assert len(c.groups) == 2
    ring = [g for g in c.groups if g.ring_pages][0]
    full = [g for g in c.groups if not g.ring_pages][0]
    assert ring.ring_pages == 2 and ring.table_stride == 2          # ceil(100 / 64)
    assert full.table_stride == 8                                    # 512 / 64
    assert len(ring.k) == 2 and len(full.k) == 2
    assert ring.k[0].data_ptr() != ring.k[1].data_ptr() != full.k[0].data_ptr()
    assert c.stores[0].kv.ring_pages == 2 and c.stores[1].kv.ring_pages == 0
    assert c.stores[0].kv.page_table.data_ptr() == c.stores[2].kv.page_table.data_ptr()
    assert c.stores[0].kv.k_pages.data_ptr() != c.stores[2].kv.k_pages.data_ptr()


def test_pages_follow_the_length_and_come_back():
    c = make()
    ring, full = (c.groups[0], c.groups[1]) if c.groups[0].ring_pages else (c.groups[1], c.groups[0])
    s = c.admit([0])[0]
    c.extend(s, 1)
    assert (full.pages.n_held, ring.pages.n_held) == (1, 1)
    c.extend(s, 64)
    assert (full.pages.n_held, ring.pages.n_held) == (1, 1)
    c.extend(s, 65)
    assert (full.pages.n_held, ring.pages.n_held) == (2, 2)
    c.extend(s, 300)
    assert (full.pages.n_held, ring.pages.n_held) == (5, 2)          # the ring stops growing
    c.check()
    c.release(s)
    assert (full.pages.n_held, ring.pages.n_held, c.slots.n_held) == (0, 0, 0)
    with pytest.raises(CacheError, match="freed twice"):
        c.release(s)
    c.check()


def test_capacity_is_max_tokens_rounded_to_pages():
    c = make(max_tokens=64 * 5, max_seq_len=4096)
    a, b = c.admit([0, 0])
    c.extend(a, 128)
    c.extend(b, 129)                      # 2 + 3 pages: full
    with pytest.raises(CacheError, match="no free page"):
        c.extend(a, 129)
    c.release(b)
    c.extend(a, 320)                      # all five pages
    with pytest.raises(CacheError, match="longer than the cache holds"):
        c.extend(a, 321)
    c.release(a)
    c.check()


def test_freed_slots_and_pages_are_used_again():
    c = make()
    first = c.admit([0, 0, 0])
    for s in first:
        c.extend(s, 70)
    pages_first = {p for g in c.groups for pages in g._slot_pages.values() for p in pages}
    c.release(first[1])
    again = c.admit([0])[0]
    assert again == first[1]
    c.extend(again, 70)
    pages_now = {p for g in c.groups for pages in g._slot_pages.values() for p in pages}
    assert pages_now == pages_first
    c.check()


def test_too_long_sequence_and_unknown_slot():
    c = make(max_tokens=4096, max_seq_len=128)
    s = c.admit([0])[0]
    with pytest.raises(CacheError, match="longer than the cache holds"):
        c.extend(s, 129)
    with pytest.raises(CacheError, match="holds no sequence"):
        c.extend(99, 1)


def test_state_is_zeroed_when_a_slot_is_taken():
    needs = [None, KVNeed(1, 16, None)]
    c = CacheManager(needs, [None, None], [[StateNeed("acc", (4,))], []], 256, 128, torch.float32, CPU)
    assert c.stores[0].kv is None and c.stores[1].kv is not None
    s = c.admit([0])[0]
    c.stores[0].state["acc"][s] += 3.0
    c.release(s)
    s2 = c.admit([0])[0]
    assert s2 == s and float(c.stores[0].state["acc"][s2].abs().sum()) == 0.0


def test_an_entry_can_read_another_entrys_cache():
    needs = [KVNeed(1, 16, None), KVNeed(1, 16, None), KVNeed(1, 16, None)]
    c = CacheManager(needs, [None, 0, None], [[], [], []], 256, 128, torch.float32, CPU)
    assert c.groups[0].n_entries == 2                     # two stores, three entries
    assert c.stores[1].kv.k_pages.data_ptr() == c.stores[0].kv.k_pages.data_ptr()
    assert c.stores[0].owns_kv and not c.stores[1].owns_kv and c.stores[2].owns_kv
    with pytest.raises(CacheError, match="another shape"):
        CacheManager([KVNeed(1, 16, None), KVNeed(2, 16, None)], [None, 0], [[], []], 256, 128,
                     torch.float32, CPU)


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    c = make(max_tokens=64 * 40, window=130, max_seq_len=1000)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.3 and c.slots.n_free:
            try:
                s = c.admit([0])[0]
                live[s] = 0
            except CacheError:
                pass
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.choice([1, 1, 1, 17, 64, 200])
            try:
                c.extend(s, n)
                live[s] = n
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        c.check()
        assert c.lengths == live
        for g in c.groups:
            for s, n in live.items():
                assert len(g._slot_pages[s]) == g.pages_for(n)
                assert g.table_host[s, : len(g._slot_pages[s])].tolist() == g._slot_pages[s]
    for s in list(live):
        c.release(s)
    c.check()
    assert all(g.pages.n_held == 0 for g in c.groups)


def test_changed_table_rows_reach_the_device_copy():
    """`flush` copies the rows that changed, neighbours in one copy, others on their own: the device
    copy of every table equals the host's afterwards, for slots taken in any order and reused."""
    c = make(max_tokens=4096, max_seq_len=512)
    rng = random.Random(3)
    slots = c.admit([0] * 9)
    for s in slots:
        c.extend(s, rng.randrange(1, 400))
    c.flush()
    for g in c.groups:
        assert torch.equal(g.table_dev, g.table_host) and not g._dirty
    # rows 1, 2, 3 and 7 change (a run and a single row); 5 is given back and taken again
    for s in (slots[1], slots[2], slots[3], slots[7]):
        c.extend(s, 500)
    c.release(slots[5])
    again = c.admit([0])[0]
    c.extend(again, 130)
    c.flush()
    for g in c.groups:
        assert torch.equal(g.table_dev, g.table_host) and not g._dirty
    c.flush()                                  # nothing changed: nothing to do
    c.check()


def test_a_ring_is_made_for_the_tokens_a_step_adds():
    # window 100: one more token per step needs 100 positions (2 pages, room 29);
    # 130 more need 229 positions (4 pages, room 157)
    c = make(chunk_tokens=1)
    assert c.chunk_room() == 2 * 64 - 100 + 1
    c = make(chunk_tokens=130)
    ring = [g for g in c.groups if g.ring_pages][0]
    assert ring.ring_pages == 4 and c.chunk_room() == 4 * 64 - 100 + 1 >= 130
    # a window that is a multiple of the page: exactly one token of room, as decoding needs
    c = make(window=128, chunk_tokens=1)
    assert c.chunk_room() == 1
    # no window anywhere: any number of tokens
    needs = [KVNeed(2, 16, None)]
    c = CacheManager(needs, [None], [[]], 256, 256, torch.float32, CPU)
    assert c.chunk_room() is None


def test_extending_the_sequences_of_a_step_is_all_or_nothing():
    c = make(max_tokens=256, max_seq_len=256)                 # 4 pages per group
    a, b, d = c.admit([0, 0, 0])
    c.extend_all([a, b], [10, 70])                            # 1 + 2 pages
    before = {s: (c.lengths[s], [list(g._slot_pages[s]) for g in c.groups]) for s in (a, b, d)}
    with pytest.raises(CacheError, match="no free pages"):
        c.extend_all([a, d], [20, 65])                        # a fits in its page, d wants 2 of the 1 left
    with pytest.raises(CacheError, match="longer than the cache holds"):
        c.extend_all([a, d], [20, 257])
    with pytest.raises(CacheError, match="holds no sequence"):
        c.extend_all([a, 99], [20, 5])
    assert before == {s: (c.lengths[s], [list(g._slot_pages[s]) for g in c.groups]) for s in (a, b, d)}
    c.check()
    c.extend_all([a, d], [20, 64])
    assert c.lengths[a] == 20 and c.lengths[d] == 64
    c.check()


def test_a_model_that_keeps_no_keys_is_not_sized_by_pages():
    # mixers with state of fixed size only: slots are counted, not derived from pages; no bound on tokens
    c = CacheManager([None, None], [None, None], [[StateNeed("s", (4,))], []], 64, 100000, torch.float32, CPU)
    assert c.n_slots == 256 and c.max_seq_len == 100000 and not c.groups
    assert c.page_tokens == 1 and c.tokens_capacity() > 10 ** 15 and c.chunk_room() is None
    slots = c.admit([0] * 200)
    c.extend_all(slots, [50000] * 200)
    assert c.stores[0].state["s"].shape == (256, 4)
    for s in slots:
        c.release(s)
    c.check()
    c = CacheManager([None], [None], [[]], 64, 1000, torch.float32, CPU, max_slots=3)
    assert c.n_slots == 3
    # with keys to keep, as before
    assert make().page_tokens == 64 and make().tokens_capacity() == 1024
