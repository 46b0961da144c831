"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice."""
import numpy as np
import pytest
import torch

from rust_inference_b200.cache import Cache, CacheError, PageTable, SlotAllocator
from rust_inference_b200.parts import CacheRequest


def test_slots_are_reused_and_never_double_freed():
    a = SlotAllocator(3)
    s = [a.alloc(), a.alloc(), a.alloc()]
    assert sorted(s) == [0, 1, 2]
    with pytest.raises(CacheError):
        a.alloc()
    a.free(s[1])
    with pytest.raises(CacheError):
        a.free(s[1])                      # freed twice
    with pytest.raises(CacheError):
        a.free(7)
    assert a.alloc() == s[1]              # the freed slot is used again
    a.check()


def test_pages_follow_the_reference_rules():
    # lazy mapping, lowest page first, over-capacity errors (src/kvcache.rs:216-247 there)
    t = PageTable(num_slots=2, num_pages=4, max_pages_per_seq=3, page_size=32)
    assert t.extend(0, 1) == 0 and t.table[0].tolist() == [0, -1, -1]
    t.extend(0, 31)
    assert t.free_pages == 3
    assert t.extend(0, 1) == 32 and t.table[0].tolist() == [0, 1, -1]      # crosses a page boundary
    with pytest.raises(CacheError, match="per sequence"):
        t.extend(0, 64)
    t.extend(1, 64)
    with pytest.raises(CacheError, match="out of pages"):
        t.extend(0, 32)
    assert t.lens == [33, 64]                                               # a failed extend changed nothing
    t.release(1)
    assert t.extend(0, 32) == 33 and t.free_pages == 1
    t.check()


def test_window_group_gives_pages_back():
    t = PageTable(num_slots=1, num_pages=4, max_pages_per_seq=100, page_size=32, window=40)
    total = 0
    for _ in range(50):
        t.extend(0, 17)
        total += 17
        t.release_behind_window(0)
        first_needed = total - 40 + 1
        row = t.table[0]
        for p in range(-(-total // 32)):
            needed = (p + 1) * 32 > first_needed
            assert (row[p] >= 0) == needed, (total, p)
        t.check()
    assert t.free_pages >= 1          # 40 keys never need more than three pages


def _cache(**kw):
    reqs = [CacheRequest(kv_heads=2, head_dim=16), CacheRequest(kv_heads=2, head_dim=16),
            CacheRequest(kv_heads=1, head_dim=32, window=8), CacheRequest(state_shape=(4,))]
    return Cache(reqs, num_slots=4, num_pages=8, max_pages_per_seq=4, dtype=torch.float32, device="cpu", **kw)


def test_groups_and_state():
    c = _cache()
    assert len(c.groups) == 2 and c.groups[0].k.shape == (2, 8, 2, 32, 16) and c.groups[1].k.shape == (1, 8, 1, 32, 32)
    a, b = c.layer(0), c.layer(1)
    assert a.page_table is b.page_table and a.k_pool.data_ptr() != b.k_pool.data_ptr()
    assert c.layer(2).page_table is not a.page_table
    st = c.layer(3)
    assert st.k_pool is None and st.state.shape == (4, 4)
    s = c.alloc_slot()
    c.state[3][s] += 5.0
    c.free_slot(s)
    assert c.alloc_slot() == s and float(c.state[3][s].abs().sum()) == 0.0   # state is zeroed on reuse


def test_random_walk_keeps_every_invariant():
    rng = np.random.default_rng(0)
    c = _cache()
    live = {}
    for step in range(600):
        r = rng.random()
        if r < 0.25 and len(live) < 4:
            live[c.alloc_slot()] = 0
        elif r < 0.4 and live:
            s = list(live)[rng.integers(len(live))]
            c.free_slot(s)
            del live[s]
            with pytest.raises(CacheError):
                c.free_slot(s)
        elif live:
            grow = [(s, int(rng.integers(1, 40))) for s in live if rng.random() < 0.7]
            if not grow:
                continue
            try:
                before = c.extend(grow)
            except CacheError:
                assert {s: c.length(s) for s in live} == live          # all or nothing
                continue
            for (s, n), b in zip(grow, before):
                assert b == live[s]
                live[s] += n
            c.upload()
            for g in c.groups:            # the copy for the kernels holds every row that changed, freed slots' too
                assert np.array_equal(g.table_dev.numpy(), g.pages.table)
            c.after_step([s for s, _ in grow])
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            full = c.groups[0].pages
            assert (full.table[s] >= 0).sum() == -(-n // 32)
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert c.free_pages() == 8 and c.slots.live_count == 0


def test_misuse():
    c = _cache()
    with pytest.raises(CacheError):
        c.extend([(0, 1)])                # slot never given out
    s = c.alloc_slot()
    with pytest.raises(CacheError):
        c.extend([(s, 0)])
    with pytest.raises(CacheError):
        c.extend([(s, 1), (s, 1)])
    with pytest.raises(CacheError):
        c.extend([(s, 4 * 32 + 1)])


def test_sizes_that_make_no_cache_are_refused():
    with pytest.raises(CacheError):
        SlotAllocator(0)
    with pytest.raises(CacheError):
        PageTable(num_slots=2, num_pages=0, max_pages_per_seq=3, page_size=32)
    with pytest.raises(CacheError):
        Cache([CacheRequest(kv_heads=1, head_dim=16)], num_slots=0, num_pages=4, max_pages_per_seq=2,
              dtype=torch.float32, device="cpu")
