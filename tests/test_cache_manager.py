"""The cache manager on the host (no GPU): pages, block tables, groups, state slots."""
import random

import numpy as np
import pytest
import torch

from vt_transformer_b200.cache import CacheManager, OutOfPages, OutOfRows, PagePool
from vt_transformer_b200.parts import KVCacheSpec, StateSpec


def manager(num_pages=8, max_requests=3, max_seq_len=128, window=None, state=False, window_pages=None):
    specs = {0: KVCacheSpec(2, 16), 1: KVCacheSpec(2, 16)}
    if window:
        specs[2] = KVCacheSpec(2, 16, window)
    if state:
        specs[9] = StateSpec((4,), torch.float32)
    return CacheManager(specs, page_size=16, num_pages=num_pages, max_requests=max_requests, max_seq_len=max_seq_len,
                        dtype=torch.float32, device="cpu", window_pages=window_pages)


def test_pool_hands_out_ascending_pages_and_refuses_double_free():
    # as vt-transformer's page table: ids come out ascending from 0 (vt-transformer/test/vt_cache_test.cpp)
    pool = PagePool(4)
    assert pool.take(3) == [0, 1, 2] and pool.free == 1
    pool.give([1])
    assert pool.take(1) == [1]            # LIFO: the page freed last is used again first
    with pytest.raises(OutOfPages):
        pool.take(5)
    assert pool.free == 1                 # all-or-nothing: nothing was taken
    pool.give([0])
    with pytest.raises(ValueError, match="twice"):
        pool.give([0])
    with pytest.raises(ValueError, match="does not belong"):
        pool.give([7])


def test_groups_by_need():
    m = manager(window=20)
    assert len(m.groups) == 2
    assert m.slot_group[0][0] == m.slot_group[1][0] != m.slot_group[2][0]
    full, win = m.groups[m.slot_group[0][0]], m.groups[m.slot_group[2][0]]
    assert full.tensors["k"].shape == (2, 8, 2, 16, 16) and win.tensors["v"].shape == (1, 8, 2, 16, 16)
    assert full.spec.window is None and win.spec.window == 20


def test_extend_commit_release_and_reuse():
    m = manager(num_pages=4)
    a = m.admit()
    m.extend([(a, 17)])                    # 2 pages
    assert m.free_pages() == [2] and list(m.groups[0].table[a, :3]) == [0, 1, -1]
    m.commit(a, 17)
    m.extend([(a, 30)])                    # still inside page 1: nothing new
    assert m.free_pages() == [2]
    m.commit(a, 30)
    b = m.admit()
    with pytest.raises(OutOfPages) as e:
        m.extend([(a, 40), (b, 33)])       # 1 + 3 pages wanted, 2 free
    assert (e.value.needed, e.value.free) == (4, 2)
    assert m.free_pages() == [2] and (m.groups[0].table[b] == -1).all()   # nothing changed
    m.extend([(b, 20)])
    m.commit(b, 20)
    assert m.free_pages() == [0]
    m.release(a)
    assert m.free_pages() == [2] and (m.groups[0].table[a] == -1).all() and m.length(a) == 0
    c = m.admit()
    assert c == a                          # the row is used again
    m.extend([(c, 32)])
    assert sorted(m.groups[0].table[c, :2]) == [0, 1]                      # and so are its pages
    m.check()
    with pytest.raises(ValueError, match="holds no request"):
        m.release(2)
    with pytest.raises(ValueError, match="max_seq_len"):
        m.extend([(c, 129)])


def test_rows_run_out():
    m = manager(max_requests=2)
    m.admit(), m.admit()
    with pytest.raises(OutOfRows):
        m.admit()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager(num_pages=6, window=20)
    full, win = m.groups[0], m.groups[1]
    r = m.admit()
    length = 0
    for step in (16, 16, 16, 1, 1, 30):
        m.extend([(r, length + step)])
        length += step
        m.commit(r, length)
        m.check()
        # a token at position >= length reads keys j > length - 20: pages below that are gone
        first = max(0, length - 20 + 1) // 16
        assert (win.table[r, :first] == -1).all()
        assert (win.table[r, first:-(-length // 16)] >= 0).all()
        assert (full.table[r, :-(-length // 16)] >= 0).all()
    assert length == 80 and full.pool.free == 1 and win.pool.free == 4
    m.release(r)
    assert full.pool.free == 6 and win.pool.free == 6
    m.check()


def test_state_slots_are_zero_on_admission():
    m = manager(state=True)
    a = m.admit()
    m.state[9][a] += 3.0
    v = m.views({0: torch.zeros(1, 1, dtype=torch.int32)})
    assert v[9].state is m.state[9] and v[0].k.shape == (8, 2, 16, 16)
    m.release(a)
    b = m.admit()
    assert b == a and float(m.state[9][b].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    """Requests admitted, extended, committed and released in random order: after every
    action no page is lost, held twice or freed twice, and a failed extend changes nothing."""
    rng = random.Random(seed)
    m = manager(num_pages=10, max_requests=4, max_seq_len=160, window=24 if seed % 2 else None,
                window_pages=6 if seed % 2 else None)
    live = {}
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.free_rows:
            live[m.admit()] = 0
        elif action < 0.85 and live:
            picks = rng.sample(sorted(live), rng.randint(1, len(live)))
            items = [(r, min(160, live[r] + rng.choice([1, 1, 2, 7, 16, 33]))) for r in picks]
            before = ([g.table.copy() for g in m.groups], m.free_pages())
            try:
                m.extend(items)
            except OutOfPages:
                assert m.free_pages() == before[1]
                assert all((g.table == t).all() for g, t in zip(m.groups, before[0]))
                victim = rng.choice(sorted(live))
                m.release(victim)
                del live[victim]
            else:
                for r, n in items:
                    m.commit(r, n)
                    live[r] = n
        elif live:
            r = rng.choice(sorted(live))
            m.release(r)
            del live[r]
        m.check()
        for r, n in live.items():
            assert m.length(r) == n
    for r in list(live):
        m.release(r)
    m.check()
    assert m.free_pages() == [g.pool.num_pages for g in m.groups] and m.free_rows == 4


def test_the_native_packing_of_a_step_equals_the_python_one():
    """The description of a step (ids, positions, offsets, rows, wanted rows, block-table rows, padding) packed by
    csrc/host_runtime.cpp and by the Python code beside it, for random mixed steps in layouts with room to spare."""
    import random

    import numpy as np

    from vt_transformer_b200.engine.batch import Layout, StepEntry, fill_host, slices_of

    rng = random.Random(4)
    m = manager(num_pages=40, max_requests=6, max_seq_len=320, window=40, window_pages=30)
    rows = [m.admit() for _ in range(5)]
    for _ in range(30):
        live = rng.sample(rows, rng.randrange(1, 6))
        entries = [StepEntry(r, [rng.randrange(1000) for _ in range(rng.choice([1, 1, 2, 7, 30]))], []) for r in live]
        entries = [e for e in entries if m.length(e.row) + len(e.tokens) <= 320]
        if not entries:
            continue
        for e in entries:
            e.want = sorted(rng.sample(range(len(e.tokens)), rng.randrange(0, min(3, len(e.tokens)) + 1)))
        m.extend([(e.row, m.length(e.row) + len(e.tokens)) for e in entries])
        seqs = slices_of(entries, m)
        want_flat = [sl.offset + w for e, sl in zip(entries, seqs) for w in e.want]
        T = sum(len(e.tokens) for e in entries)
        lay = Layout.make(T + rng.randrange(0, 5), len(entries) + rng.randrange(0, 3), len(want_flat) + rng.randrange(0, 3),
                          m.max_pages, len(m.groups))
        native = np.full(lay.total, 12345, dtype=np.int32)
        fill_host(native, lay, entries, seqs, want_flat, m)

        class NoBook:                      # the same manager without its C++ side: the Python packing
            page_size, groups = m.page_size, m.groups
            table_rows = staticmethod(m.table_rows)
        plain = np.full(lay.total, 12345, dtype=np.int32)
        fill_host(plain, lay, entries, seqs, want_flat, NoBook)
        for i in range(len(lay.sizes)):
            assert (lay.seg(native, i) == lay.seg(plain, i)).all(), i
        for e in entries:
            m.commit(e.row, m.length(e.row) + len(e.tokens))
        if rng.random() < 0.2:
            r = rng.choice(rows)
            m.release(r)
            rows[rows.index(r)] = m.admit()
    m.check()
