"""The cache's bookkeeping on the host: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from quicknn_b200.cache import PAGE, CacheFull, KVCache, PagePool, SlotTable
from quicknn_b200.parts import CacheNeed, StateNeed


def make(max_tokens=512, max_slots=4, max_seq=256, window=8):
    needs = [CacheNeed(2, 16, window), CacheNeed(2, 16, None), CacheNeed(2, 16, window), CacheNeed(2, 16, None)]
    return KVCache(needs, [None] * 4, max_tokens, max_slots, max_seq, torch.float32, "cpu")


def test_pool_invariants():
    p = PagePool(5)
    a = p.take(3)
    assert a == [1, 2, 3] and p.n_free == 1
    with pytest.raises(CacheFull):
        p.take(2)
    p.give_back([2])
    with pytest.raises(RuntimeError):
        p.give_back([2])                       # freed twice
    with pytest.raises(ValueError):
        p.give_back([0])                       # page 0 is never handed out
    assert p.take(2) == [2, 4]
    p.audit()


def test_slot_table():
    t = SlotTable(2)
    assert (t.take(), t.take()) == (0, 1)
    with pytest.raises(CacheFull):
        t.take()
    t.give_back(0)
    with pytest.raises(RuntimeError):
        t.give_back(0)
    assert t.take() == 0                       # used again at once


def test_groups_have_storage_of_their_own():
    c = make()
    assert len(c.groups) == 2
    local = [g for g in c.groups if g.ring][0]
    full = [g for g in c.groups if not g.ring][0]
    assert local.ring == PAGE and local.pages_per_seq == 1 and local.lines == [0, 2]
    assert full.pages_per_seq == 4 and full.lines == [1, 3]
    assert c.line(0).k.data_ptr() != c.line(2).k.data_ptr() != c.line(1).k.data_ptr()
    assert tuple(c.line(1).k.shape) == (512 // PAGE + 1, 2, PAGE, 16)
    assert c.line(0).ring == PAGE and c.line(1).ring == 0


def test_extend_free_reuse_and_limits():
    c = make(max_tokens=256, max_slots=3, max_seq=200)
    a, b = c.allocate(), c.allocate()
    c.extend([(a, 70), (b, 5)])
    c.audit()
    assert c.length(a) == 70 and c.tokens_held() == 128 + 64
    full = [g for g in c.groups if not g.ring][0]
    local = [g for g in c.groups if g.ring][0]
    assert len(full.held[a]) == 2 and len(local.held[a]) == 1 and len(full.held[b]) == 1
    with pytest.raises(CacheFull):             # 70 -> 200 needs 2 more pages, only 1 is free
        c.extend([(a, 200)])
    assert c.length(a) == 70                   # nothing changed
    c.audit()
    with pytest.raises(CacheFull):
        c.extend([(b, 201)])                   # beyond the longest sequence
    with pytest.raises(ValueError):
        c.extend([(a, 10)])                    # cannot shrink
    pages_a = list(full.held[a])
    c.free(a)
    with pytest.raises(RuntimeError):
        c.free(a)                              # freed twice
    with pytest.raises(RuntimeError):
        c.extend([(a, 3)])                     # not in use
    c.audit()
    d = c.allocate()
    assert d == a                              # the slot is used again
    c.extend([(d, 128)])
    assert sorted(full.held[d]) == sorted(pages_a)      # and so are its pages
    c.extend([(b, 64)])
    with pytest.raises(CacheFull):
        c.extend([(b, 129)])                   # the pool is exhausted: 2 + 3 > 4 pages
    c.audit()


def test_all_or_nothing_across_sequences():
    c = make(max_tokens=192, max_slots=3, max_seq=192)
    a, b = c.allocate(), c.allocate()
    with pytest.raises(CacheFull):
        c.extend([(a, 100), (b, 100)])         # 2 + 2 pages of 3
    assert c.length(a) == 0 and c.length(b) == 0
    c.audit()
    c.extend([(a, 100), (b, 60)])
    c.audit()


def test_random_walk_keeps_invariants():
    rnd = random.Random(0)
    c = make(max_tokens=1024, max_slots=6, max_seq=400)
    live = {}
    for _ in range(600):
        r = rnd.random()
        if r < 0.25 and len(live) < 6:
            live[c.allocate()] = 0
        elif r < 0.45 and live:
            s = rnd.choice(list(live))
            c.free(s)
            del live[s]
        elif r < 0.55 and live:
            s = rnd.choice(list(live))                      # the undo of a step that was not launched
            live[s] = max(0, live[s] - rnd.choice([1, 1, 17, 90]))
            c.truncate([(s, live[s])])
        elif live:
            s = rnd.choice(list(live))
            n = live[s] + rnd.choice([1, 1, 1, 17, 90])
            try:
                c.extend([(s, n)])
                live[s] = n
            except CacheFull:
                pass
        c.audit()
        assert {s: c.length(s) for s in live} == live
        assert c.tokens_held() <= c.max_tokens
    for s in list(live):
        c.free(s)
    c.audit()
    assert all(g.pool.n_held == 0 for g in c.groups)


def test_state_region_zeroed_on_allocation():
    c = KVCache([CacheNeed(1, 8, None), None], [None, StateNeed((3, 2), "float32")], 128, 2, 128,
                torch.float32, "cpu")
    assert c.line(0).state is None
    st = c.line(1).state
    assert tuple(st.shape) == (2, 3, 2) and c.line(1).k is None
    s = c.allocate()
    st[s] += 5.0
    c.free(s)
    s2 = c.allocate()
    assert s2 == s and float(c.line(1).state[s2].abs().sum()) == 0.0
    empty = make()
    assert empty.state == {}                  # Gemma 2 asks for no state: zero lines


def test_truncate_gives_back_what_extend_took():
    c = make(max_tokens=512, max_slots=4, max_seq=256, window=100)
    a = c.allocate()
    c.extend([(a, 70)])
    free = [g.pool.n_free for g in c.groups]
    c.extend([(a, 200)])
    c.truncate([(a, 70)])
    assert c.length(a) == 70 and [g.pool.n_free for g in c.groups] == free
    c.audit()
    with pytest.raises(ValueError):
        c.truncate([(a, 71)])
    c.truncate([(a, 0)])
    assert c.tokens_held() == 0
    c.audit()


def test_a_windowed_group_holds_a_ring_per_slot_at_most():
    c = make(max_tokens=4096, max_slots=2, max_seq=2048, window=100)
    ring_group = [g for g in c.groups if g.ring][0]
    full_group = [g for g in c.groups if not g.ring][0]
    assert ring_group.ring == 128 and ring_group.pool.n_pages == 2 * 2 + 1
    assert full_group.pool.n_pages == 4096 // PAGE + 1
    a, b = c.allocate(), c.allocate()
    c.extend([(a, 2048), (b, 2048)])               # both rings full, the pool of the ring group exhausted
    assert ring_group.pool.n_free == 0
    c.audit()


def test_how_far_a_sequence_can_go_back():
    """A ring of 128 positions for a window of 100: once later tokens have overwritten earlier ones, a sequence of L
    tokens can be shortened by 128 - 100 + 1 at most; before that, and in groups that keep everything, to any length;
    with fixed-size state not at all."""
    c = make(max_tokens=4096, max_slots=2, max_seq=2048, window=100)
    a = c.allocate()
    c.extend([(a, 90)])
    assert c.rewind_limit(a) == 0
    c.extend([(a, 128)])
    assert c.rewind_limit(a) == 0                  # nothing overwritten yet
    c.extend([(a, 129)])
    assert c.rewind_limit(a) == 129 - 29           # position 0 is gone: the next query needs positions >= P - 99
    c.extend([(a, 1000)])
    assert c.rewind_limit(a) == 971
    c.truncate([(a, 971)])
    assert c.rewind_limit(a) == 971                # what the ring lost when the sequence was 1000 long stays lost
    c.extend([(a, 990)])
    assert c.rewind_limit(a) == 971
    c.free(a)
    a = c.allocate()
    c.extend([(a, 50)])
    assert c.rewind_limit(a) == 0                  # a new sequence in the slot starts over
    full = KVCache([CacheNeed(2, 16, None)], [None], 512, 2, 256, torch.float32, "cpu")
    b = full.allocate()
    full.extend([(b, 200)])
    assert full.rewind_limit(b) == 0
    st = KVCache([CacheNeed(1, 8, None), None], [None, StateNeed((3, 2), "float32")], 128, 2, 128, torch.float32, "cpu")
    s = st.allocate()
    st.extend([(s, 40)])
    assert st.rewind_limit(s) == 40


def test_the_device_copies_can_be_checked_against_the_host():
    c = make()
    a = c.allocate()
    c.extend([(a, 100)])
    c.verify_device()                              # on the CPU the "device" copies are plain tensors
    c.groups[0].table_dev[a, 0] += 1
    with pytest.raises(AssertionError):
        c.verify_device()

