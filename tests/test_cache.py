"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from ghost_infer_b200.cache import (PAGE_TOKENS, CacheFullError, CacheRequest, PagePool, SequenceCache, SlotAllocator,
                                    StateRequest, pages_for)


def make_cache(max_tokens=1024, max_slots=8, window=None, state=False, layers=3):
    req = CacheRequest("window", 2, 16, window) if window else CacheRequest("full", 2, 16)
    requests = [(i, req, StateRequest((4,)) if state else None, None) for i in range(layers)]
    return SequenceCache(requests, max_tokens=max_tokens, max_slots=max_slots, max_seq_len=4096,
                         dtype=torch.float32, device="cpu")


def test_pool_never_hands_a_page_twice():
    pool = PagePool(10)
    a = pool.take(4)
    b = pool.take(6)
    assert sorted(a + b) == list(range(1, 11)) and 0 not in a + b
    with pytest.raises(CacheFullError):
        pool.take(1)
    pool.give_back(a)
    with pytest.raises(RuntimeError):
        pool.give_back(a)            # freed twice
    with pytest.raises(RuntimeError):
        pool.give_back([0])          # the trash page is nobody's
    assert pool.free_pages == 4


def test_slots_lowest_first_and_no_double_free():
    s = SlotAllocator(3)
    assert [s.take(), s.take(), s.take()] == [0, 1, 2]
    with pytest.raises(CacheFullError):
        s.take()
    s.give_back(1)
    with pytest.raises(RuntimeError):
        s.give_back(1)
    assert s.take() == 1 and s.live_slots() == [0, 1, 2]


def test_reserve_commit_close_accounting():
    c = make_cache(max_tokens=640)      # 10 pages
    a, b = c.open_slot(), c.open_slot()
    c.reserve([(a, 65), (b, 64)])
    assert c.free_pages == 10 - 3
    c.commit(a, 65)
    c.commit(b, 64)
    c.reserve([(a, 66), (b, 65)])       # a stays within its second page, b needs one more
    assert c.free_pages == 10 - 4
    g = c.groups[0]
    assert len(set(g.pages[a]) | set(g.pages[b])) == 4 and 0 not in g.pages[a] + g.pages[b]
    assert list(g.table_host[a, :2]) == g.pages[a] and list(g.table_host[b, :2]) == g.pages[b]
    c.close_slot(a)
    assert c.free_pages == 10 - 2
    with pytest.raises(RuntimeError):
        c.close_slot(a)
    c.close_slot(b)
    assert c.free_pages == 10 and c.slots.free_slots == 8


def test_reserve_is_all_or_nothing():
    c = make_cache(max_tokens=256)      # 4 pages
    a, b = c.open_slot(), c.open_slot()
    with pytest.raises(CacheFullError):
        c.reserve([(a, 128), (b, 192)])
    assert c.free_pages == 4 and c.groups[0].pages[a] == []
    c.reserve([(a, 128), (b, 128)])
    assert c.free_pages == 0


def test_context_full_per_slot():
    req = CacheRequest("full", 1, 16)
    c = SequenceCache([(0, req, None, None)], max_tokens=4096, max_slots=2, max_seq_len=100, dtype=torch.float32)
    s = c.open_slot()
    with pytest.raises(CacheFullError) as e:
        c.reserve([(s, 101)])
    assert "context full" in str(e.value)


def test_random_churn_conserves_pages():
    rnd = random.Random(0)
    c = make_cache(max_tokens=64 * 40, max_slots=6)
    live = {}
    for _ in range(600):
        op = rnd.random()
        if op < 0.3 and c.slots.free_slots:
            live[c.open_slot()] = 0
        elif op < 0.75 and live:
            s = rnd.choice(list(live))
            n = live[s] + rnd.randint(1, 150)
            try:
                c.reserve([(s, n)])
                c.commit(s, n)
                live[s] = n
            except CacheFullError:
                pass
        elif live:
            s = rnd.choice(list(live))
            c.close_slot(s)
            del live[s]
        g = c.groups[0]
        held = [p for s in live for p in g.pages[s]]
        assert len(held) == len(set(held)) and 0 not in held           # no page held twice
        assert len(held) + c.free_pages == 40                         # none lost
        assert all(len(g.pages[s]) >= pages_for(live[s]) for s in live)
        assert sorted(c.slots.live_slots()) == sorted(live)


def test_window_group_gives_pages_back_early():
    c = make_cache(max_tokens=64 * 20, window=100)
    s = c.open_slot()
    n = 0
    for _ in range(500):
        n += 1
        c.reserve([(s, n)])
        c.commit(s, n)
    g = c.groups[0]
    live = [p for p in g.pages[s] if p != 0]
    # positions below n - window + 1 = 401 are dead: page indices 0..5 (tokens 0..383) are released
    assert g.first_live[s] == 401 // PAGE_TOKENS == 6
    assert len(live) == pages_for(500) - 6 and c.free_pages == 20 - len(live)
    c.close_slot(s)
    assert c.free_pages == 20


def test_groups_by_request_and_shared_memory():
    full, win = CacheRequest("full", 2, 16), CacheRequest("window", 2, 16, 32)
    reqs = [(0, full, None, None), (1, win, None, None), (2, full, None, None), (3, None, None, 0), (4, None, StateRequest((3, 2)), None)]
    c = SequenceCache(reqs, max_tokens=256, max_slots=4, max_seq_len=256, dtype=torch.float32)
    assert len(c.groups) == 2 and c.groups[0].k.shape == (2, 5, 2, PAGE_TOKENS, 16) and c.groups[1].k.shape[0] == 1
    m0, m3, m4 = c.memory(0), c.memory(3), c.memory(4)
    assert m3.k.data_ptr() == m0.k.data_ptr() and m0.writes and not m3.writes      # entry 3 reads entry 0's cache
    assert c.memory(1).window == 32 and m0.window is None
    assert m4.k is None and m4.state.shape == (4 + 1, 3, 2)          # four slots and the padding rows' trash row
    assert c.bytes_per_token() == 2 * 3 * 2 * 16 * 4 and c.state_bytes_per_sequence() == 24


def test_state_is_zeroed_when_a_slot_opens():
    c = make_cache(state=True)
    s = c.open_slot()
    c.memory(0).state[s] += 5.0
    c.close_slot(s)
    s2 = c.open_slot()
    assert s2 == s and float(c.memory(0).state[s2].abs().sum()) == 0.0


def test_truncate_rewinds_and_frees():
    c = make_cache(max_tokens=640)
    s = c.open_slot()
    c.reserve([(s, 200)])
    c.commit(s, 200)
    assert c.truncate(s, 70) == 70 and c.free_pages == 10 - 2 and c.length(s) == 70
    cs = make_cache(state=True)
    s = cs.open_slot()
    cs.reserve([(s, 10)])
    cs.commit(s, 10)
    assert cs.truncate(s, 5) == 10          # fixed-size state cannot be rewound


def test_reset_starts_a_slot_over():
    c = make_cache(max_tokens=640, state=True)
    s = c.open_slot()
    c.reserve([(s, 200)])
    c.commit(s, 200)
    c.memory(0).state[s] += 3.0
    c.reset(s)
    assert c.length(s) == 0 and c.free_pages == 10 and float(c.memory(0).state[s].abs().sum()) == 0.0
    assert c.slots.live(s)
    c.reserve([(s, 65)])
    assert c.free_pages == 8
    with pytest.raises(RuntimeError):
        c.reset(s + 1)
