"""The cache's bookkeeping: no slot or page lost, held twice or freed twice;
groups with storage of their own; windows give pages back."""
import random

import pytest

from esp_b200.cache import PAGE, CacheBook, FreeList, KvLayout, pages_for
from esp_b200.errors import CacheFull, InvalidRequest

FULL = KvLayout(2, 16, None)
WIN = KvLayout(2, 16, 100)


def test_free_list_hands_each_id_to_one_owner():
    f = FreeList(5, "slot")
    got = f.take(5)
    assert sorted(got) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        f.take(1)
    f.give_back([got[2]])
    with pytest.raises(InvalidRequest):
        f.give_back([got[2]])             # freed twice
    with pytest.raises(InvalidRequest):
        f.give_back([99])                 # never taken
    assert f.take(1) == [got[2]]          # the id given back last is used again first
    with pytest.raises(InvalidRequest):
        f.give_back([got[0], got[0]])


def test_slots_are_reused_and_lengths_tracked():
    book = CacheBook([FULL], max_tokens=10 * PAGE, max_slots=3, max_positions=1000)
    a, b, c = book.open(), book.open(), book.open()
    with pytest.raises(CacheFull):
        book.open()
    book.reserve({a: 70, b: 1})
    book.commit({a: 70, b: 1})
    assert book.length(a) == 70 and book.length(b) == 1 and book.length(c) == 0
    assert book.groups[0].pool.available == 10 - 3
    book.close(b)
    with pytest.raises(InvalidRequest):
        book.close(b)
    with pytest.raises(InvalidRequest):
        book.length(b)
    d = book.open()
    assert d == b and book.length(d) == 0
    assert book.groups[0].pool.available == 10 - 2


def test_step_is_refused_whole_when_it_does_not_fit():
    book = CacheBook([FULL], max_tokens=4 * PAGE, max_slots=4, max_positions=1000)
    a, b = book.open(), book.open()
    with pytest.raises(CacheFull):
        book.reserve({a: 3 * PAGE, b: PAGE + 1})
    assert book.groups[0].pool.available == 4 and book.groups[0].tables == {}
    with pytest.raises(InvalidRequest):
        book.reserve({a: 1001})
    with pytest.raises(InvalidRequest):
        book.reserve({a: 0})
    book.reserve({a: 3 * PAGE, b: PAGE})
    assert book.groups[0].pool.available == 0


def test_pages_are_never_shared_and_all_come_back():
    rng = random.Random(0)
    book = CacheBook([FULL, WIN], max_tokens=64 * PAGE, max_slots=8, max_positions=100000)
    live = {}
    for _ in range(400):
        if live and (rng.random() < 0.3 or len(live) == 8):
            s = rng.choice(list(live))
            book.close(s)
            del live[s]
        elif rng.random() < 0.5 and len(live) < 8:
            live[book.open()] = 0
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 5, 64, 130])
            try:
                book.reserve({s: n})
            except CacheFull:
                continue
            book.commit({s: n})
            live[s] += n
        for g in book.groups:
            held = [p for t in g.tables.values() for p in t if p >= 0]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + g.pool.available == g.pool.n, "a page was lost"
        for s, n in live.items():
            assert book.length(s) == n
            full = book.groups[0].tables.get(s, [])
            assert sum(p >= 0 for p in full) == pages_for(n)
    for s in list(live):
        book.close(s)
    assert all(g.pool.available == g.pool.n and not g.tables for g in book.groups)
    assert book.slots.available == 8


def test_window_group_gives_pages_back_but_keeps_what_queries_see():
    book = CacheBook([FULL, KvLayout(1, 8, 70)], max_tokens=40 * PAGE, max_slots=2, max_positions=10000)
    s = book.open()
    book.reserve({s: 300})
    assert sum(p >= 0 for p in book.groups[1].tables[s]) == pages_for(300)   # a prompt needs all its pages
    book.commit({s: 300})
    # the next query (position 300) sees positions 231..300: pages 3 and 4
    t = book.groups[1].tables[s]
    assert [p >= 0 for p in t] == [False, False, False, True, True]
    assert sum(p >= 0 for p in book.groups[0].tables[s]) == 5                # the full group keeps everything
    for _ in range(200):
        book.reserve({s: 1})
        book.commit({s: 1})
        n = book.length(s)
        t = book.groups[1].tables[s]
        first = max(0, n - 70 + 1)
        for pos in range(first, n):
            assert t[pos // PAGE] >= 0
        assert sum(p >= 0 for p in t) <= 3
    book.close(s)
    assert book.groups[1].pool.available == 40


def test_table_rows_are_padded_for_the_device():
    book = CacheBook([FULL], max_tokens=8 * PAGE, max_slots=2, max_positions=1000)
    a, b = book.open(), book.open()
    book.reserve({a: 130, b: 3})
    rows = book.groups[0].table_rows([a, b], 4)
    assert len(rows[0]) == 4 and rows[0][3] == -1 and rows[0][2] >= 0 and rows[1][1:] == [-1, -1, -1]
    with pytest.raises(InvalidRequest):
        book.groups[0].table_rows([a], 2)


def test_a_cancelled_reservation_gives_every_page_back_and_leaves_the_tables_as_they_were():
    """A step whose forward pass fails: the pages it took go back, lengths and tables stay, in a group that
    keeps everything and in one with a window whose table has gaps."""
    rng = random.Random(3)
    book = CacheBook([FULL, WIN], max_tokens=40 * PAGE, max_slots=4, max_positions=5000)
    a, b = book.open(), book.open()
    first = {a: 300, b: 70}
    book.reserve(first)
    book.commit(first)
    for _ in range(200):
        growth = {a: rng.choice([1, 1, 1, 64, 130]), b: rng.choice([1, 2, 65])}
        free = [g.pool.available for g in book.groups]
        tables = [{s: list(t) for s, t in g.tables.items()} for g in book.groups]
        lengths = dict(book.lengths)
        try:
            receipts = book.reserve(growth)
        except CacheFull:
            break
        if rng.random() < 0.5:
            book.cancel(receipts)
            assert [g.pool.available for g in book.groups] == free
            assert [{s: list(t) for s, t in g.tables.items()} for g in book.groups] == tables
            assert book.lengths == lengths
        else:
            book.commit(growth)
    book.close(a)
    book.close(b)
    assert all(g.pool.available == g.pool.n for g in book.groups) and book.slots.available == 4
