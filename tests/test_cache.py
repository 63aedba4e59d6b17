"""The cache's bookkeeping without a GPU: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

import qstream_b200 as qs
from qstream_b200.cache import KvNeed, PagePool, SequenceCache, SlotTable, StateNeed


def test_page_pool_hands_out_each_page_once():
    pool = PagePool(5)
    pages = [pool.alloc() for _ in range(5)]
    assert sorted(pages) == [0, 1, 2, 3, 4] and pool.n_free == 0
    with pytest.raises(qs.QStreamError) as e:
        pool.alloc()
    assert e.value.code == qs.QsError.BUDGET_EXCEEDED
    pool.free(3)
    with pytest.raises(qs.QStreamError):
        pool.free(3)                                    # freed twice
    with pytest.raises(qs.QStreamError):
        pool.free(7)                                    # never existed
    assert pool.alloc() == 3
    pool.check()


def test_slot_table_acquire_release():
    t = SlotTable(3)
    a, b, c = t.acquire(), t.acquire(), t.acquire()
    assert {a, b, c} == {0, 1, 2}
    with pytest.raises(qs.QStreamError) as e:
        t.acquire()
    assert e.value.code == qs.QsError.BUDGET_EXCEEDED
    t.length[b] = 17
    t.release(b)
    with pytest.raises(qs.QStreamError):
        t.release(b)                                    # released twice
    again = t.acquire()
    assert again == b and t.length[again] == 0 and t.generation[again] == 2
    t.check()


def make_cache(max_tokens=640, max_slots=4, ctx=256, window=0, state=False):
    needs = {0: KvNeed(2, 16, 0), 1: KvNeed(2, 16, 0), 2: KvNeed(2, 16, window)} if window else \
            {0: KvNeed(2, 16, 0), 1: KvNeed(2, 16, 0)}
    states = {5: StateNeed((3, 4), torch.float32)} if state else {}
    return SequenceCache(needs, states, max_tokens, max_slots, ctx, torch.float32, "cpu")


def test_groups_by_need_and_views():
    c = make_cache(window=100)
    assert len(c.groups) == 2                           # full and windowed layers have storage of their own
    full = [g for g in c.groups if g.need.window == 0][0]
    assert full.entries == [0, 1] and full.k.shape == (2, 10 + 1, 2, 64, 16)     # ten pages and the guard page
    v = c.view(1)
    assert v.k.shape == (11, 2, 64, 16) and v.page_table.shape == (4, 4) and v.page_tokens == 64
    assert c.view(2).need.window == 100


def test_prepare_commit_release_and_reuse():
    c = make_cache()
    a, b = c.acquire(), c.acquire()
    c.prepare([a, b], [70, 5])
    c.commit([a, b], [70, 5])
    assert c.length(a) == 70 and c.length(b) == 5
    g = c.groups[0]
    assert (g.table_host[a] >= 0).sum() == 2 and (g.table_host[b] >= 0).sum() == 1
    assert torch.equal(g.table_dev.cpu(), torch.from_numpy(g.table_host))
    for _ in range(59):
        c.prepare([a, b], [1, 1]); c.commit([a, b], [1, 1])
    assert (g.table_host[b] >= 0).sum() == 1            # 64 tokens still fit one page
    c.prepare([b], [1]); c.commit([b], [1])
    assert (g.table_host[b] >= 0).sum() == 2
    c.check()
    held = g.pool.n_pages - g.pool.n_free
    c.release(a)
    assert g.pool.n_pages - g.pool.n_free == held - 3
    with pytest.raises(qs.QStreamError):
        c.release(a)
    a2 = c.acquire()
    assert a2 == a and c.length(a2) == 0                # the slot is used again, empty
    c.check()


def test_errors_leave_the_cache_untouched():
    c = make_cache(max_tokens=256, max_slots=4, ctx=128)
    a, b = c.acquire(), c.acquire()
    with pytest.raises(qs.QStreamError) as e:
        c.prepare([a], [129])
    assert e.value.code == qs.QsError.SEQ_TOO_LONG
    with pytest.raises(qs.QStreamError) as e:
        c.prepare([a, a], [1, 1])
    assert e.value.code == qs.QsError.INVALID_INPUT
    c.prepare([a], [128]); c.commit([a], [128])
    c.prepare([b], [100]); c.commit([b], [100])         # all 4 pages in use
    d = c.acquire()
    with pytest.raises(qs.QStreamError) as e:
        c.prepare([d], [1])
    assert e.value.code == qs.QsError.BUDGET_EXCEEDED and "pages" in str(e.value)
    assert c.groups[0].pool.n_free == 0 and c.length(d) == 0
    with pytest.raises(qs.QStreamError):
        c.prepare([3], [1])                             # not acquired
    c.check()


def test_window_gives_pages_back():
    c = make_cache(max_tokens=1024, max_slots=2, ctx=1024, window=100)
    win = [g for g in c.groups if g.need.window][0]
    full = [g for g in c.groups if not g.need.window][0]
    s = c.acquire()
    c.prepare([s], [300]); c.commit([s], [300])
    # the next query (position 300) reads keys >= 201: pages 0..2 (keys < 192) are given back
    assert list(win.table_host[s][:5] >= 0) == [False, False, False, True, True]
    assert (full.table_host[s] >= 0).sum() == 5
    for _ in range(200):
        c.prepare([s], [1]); c.commit([s], [1])
    assert (win.table_host[s] >= 0).sum() == 2 and (full.table_host[s] >= 0).sum() == 8
    c.check()
    c.release(s)
    assert win.pool.n_free == win.pool.n_pages and full.pool.n_free == full.pool.n_pages


def test_state_is_zeroed_when_a_slot_is_taken():
    c = make_cache(state=True)
    s = c.acquire()
    st = c.state.get(5)
    assert st.shape == (4, 3, 4)
    st[s] += 7
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(st[s2].abs().sum()) == 0.0
    assert make_cache().state.tensors == {}             # a model without state has an empty store


def test_random_walk_keeps_the_invariants():
    rnd = random.Random(0)
    c = make_cache(max_tokens=64 * 24, max_slots=6, ctx=512, window=90)
    live = {}
    for step in range(600):
        op = rnd.random()
        if op < 0.25 and c.slots.n_free:
            live[c.acquire()] = 0
        elif op < 0.4 and live:
            s = rnd.choice(list(live)); c.release(s); del live[s]
        elif live:
            chosen = rnd.sample(list(live), rnd.randint(1, len(live)))
            n_new = [rnd.choice([1, 1, 1, 7, 64, 130]) for _ in chosen]
            try:
                c.prepare(chosen, n_new)
            except qs.QStreamError as e:
                assert e.code in (qs.QsError.SEQ_TOO_LONG, qs.QsError.BUDGET_EXCEEDED)
            else:
                c.commit(chosen, n_new)
                for s, n in zip(chosen, n_new):
                    live[s] += n
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            for g in c.groups:
                first = max(0, n - g.need.window + 1) // 64 if g.need.window else 0
                have = set((g.table_host[s] >= 0).nonzero()[0].tolist())
                assert have == set(range(first, -(-n // 64))), (s, n, g.need, have)
    for s in list(live):
        c.release(s)
    c.check()
    assert all(g.pool.n_free == g.pool.n_pages for g in c.groups)
