"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from smolmoe_c99_b200.cache import (PAGE_SIZE, CacheFull, CacheStateError, PageAllocator, SequenceCache, SlotAllocator,
                                    pages_for)
from smolmoe_c99_b200.parts import KVNeed, StateNeed


def test_slot_allocator_invariants():
    s = SlotAllocator(4)
    held = [s.alloc() for _ in range(4)]
    assert held == [0, 1, 2, 3] and s.free_count == 0
    with pytest.raises(CacheFull):
        s.alloc()
    s.free(2)
    with pytest.raises(CacheStateError, match="freed twice"):
        s.free(2)
    with pytest.raises(CacheStateError):
        s.free(7)
    assert s.alloc() == 2                      # a slot that was given back is used again
    rng = random.Random(0)
    live = set(held)
    for _ in range(500):
        if live and rng.random() < 0.5:
            x = rng.choice(sorted(live)); s.free(x); live.remove(x)
        elif len(live) < 4:
            x = s.alloc(); assert x not in live; live.add(x)
        assert s.held() == live and s.free_count == 4 - len(live)


def test_page_allocator_all_or_nothing():
    p = PageAllocator(10)
    a = p.alloc(4)
    with pytest.raises(CacheFull):
        p.alloc(7)
    assert p.free_count == 6 and p.held_count == 4      # the failed call took nothing
    b = p.alloc(6)
    assert sorted(a + b) == list(range(10))
    p.free(a)
    with pytest.raises(CacheStateError):
        p.free(a)
    with pytest.raises(CacheStateError):
        p.free([b[0], b[0] + 100])
    assert p.held_count == 6                             # a refused free changed nothing


def _cache(needs, max_tokens=1024, max_slots=4, max_seq_len=512):
    return SequenceCache(needs, max_tokens=max_tokens, max_slots=max_slots, max_seq_len=max_seq_len,
                         dtype=torch.float32, device="cpu")


def test_groups_by_need():
    full, win = KVNeed(2, 16, None), KVNeed(2, 16, 100)
    c = _cache([full, win, win, None, StateNeed((3, 5)), 0])
    assert len(c.groups) == 2 and c.groups[0].n_layers == 1 and c.groups[1].n_layers == 2
    assert c.groups[1].ring == 128 and c.groups[1].pages_per_seq == 2 and c.groups[0].pages_per_seq == 8
    v0, v1, v2, v3, v4, v5 = (c.run_view(i) for i in range(6))
    assert v0.kind == "kv" and v0.ring == 0 and v1.ring == 128 and v1.window == 100
    assert v1.k_pool.data_ptr() != v2.k_pool.data_ptr() and v1.page_table.data_ptr() == v2.page_table.data_ptr()
    assert v3.kind == "none" and v4.kind == "state" and tuple(v4.state.shape) == (4, 3, 5)
    assert v5.k_pool.data_ptr() == v0.k_pool.data_ptr()       # run 5 reads run 0's cache
    assert v0.k_pool.shape == (pages_for(1024), 2, PAGE_SIZE, 16)
    with pytest.raises(ValueError, match="owns none"):
        _cache([None, 0])
    with pytest.raises(ValueError):
        _cache([1, full])


def test_reserve_free_and_reuse():
    c = _cache([KVNeed(1, 16, None), KVNeed(1, 16, 70)], max_tokens=640, max_slots=3, max_seq_len=400)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve({a: 65, b: 300}); c.advance({a: 65, b: 300})
    full, win = c.groups
    assert len(full.slot_pages[a]) == 2 and len(full.slot_pages[b]) == 5
    assert len(win.slot_pages[a]) == 2 and len(win.slot_pages[b]) == 2      # the ring holds 128 positions
    assert full.ledger.held_count == 7 and win.ledger.held_count == 4
    before = (full.ledger.held_count, win.ledger.held_count, dict(c.lengths))
    with pytest.raises(CacheFull):
        c.reserve({a: 1, b: 101})         # b would pass 400 positions
    with pytest.raises(CacheFull):
        c.reserve({a: 300})               # 10 pages in all; 7 are held, a needs 4 more
    assert (full.ledger.held_count, win.ledger.held_count, dict(c.lengths)) == before    # all or nothing
    c.flush_tables()
    assert c.groups[0].table[b, :5].tolist() == full.slot_pages[b]
    c.free_slot(b)
    assert full.ledger.held_count == 2 and win.ledger.held_count == 2
    with pytest.raises(CacheStateError):
        c.free_slot(b)
    assert c.alloc_slot() == b and c.length(b) == 0 and full.slot_pages[b] == []
    c.free_slot(a); c.free_slot(b)
    assert full.ledger.held_count == 0 and win.ledger.held_count == 0 and c.slots.free_count == 3


def test_random_walk_never_loses_a_page():
    rng = random.Random(1)
    c = _cache([KVNeed(1, 8, None), KVNeed(1, 8, 40)], max_tokens=2048, max_slots=6, max_seq_len=700)
    live = {}
    for _ in range(400):
        r = rng.random()
        if r < 0.25 and len(live) < 6:
            live[c.alloc_slot()] = 0
        elif r < 0.45 and live:
            s = rng.choice(sorted(live)); c.free_slot(s); del live[s]
        elif live:
            s = rng.choice(sorted(live)); n = rng.randint(1, 90)
            try:
                c.reserve({s: n}); c.advance({s: n}); live[s] += n
            except CacheFull:
                pass
        for g in c.groups:
            pages = [p for s in live for p in g.slot_pages[s]]
            assert len(pages) == len(set(pages)) == g.ledger.held_count           # none held twice, none lost
            assert all(len(g.slot_pages[s]) == g.pages_needed(live[s]) for s in live)
        assert c.lengths == live
    for s in list(live):
        c.free_slot(s)
    assert all(g.ledger.held_count == 0 for g in c.groups)


def test_state_is_zeroed_when_a_slot_is_given_out():
    c = _cache([StateNeed((4,))])
    s = c.alloc_slot()
    c.run_view(0).state[s] = 7.0
    c.free_slot(s)
    assert c.alloc_slot() == s and float(c.run_view(0).state[s].abs().sum()) == 0.0


def test_truncate_rules():
    c = _cache([KVNeed(1, 8, None)])
    s = c.alloc_slot(); c.reserve({s: 100}); c.advance({s: 100})
    c.truncate(s, 40)
    assert c.length(s) == 40
    with pytest.raises(CacheStateError):
        c.truncate(s, 41)
    w = _cache([KVNeed(1, 8, 32)])
    s = w.alloc_slot(); w.reserve({s: 100}); w.advance({s: 100})
    with pytest.raises(CacheStateError, match="windowed"):
        w.truncate(s, 40)


def test_what_a_cta_that_gives_up_still_has_in_flight():
    """The bookkeeping behind the kernels' way out after a bounded wait ran out (csrc/drain.cuh), on the host: of the
    stage fills asked for, those not waited for yet, with the stage and the barrier phase each completes."""
    import ctypes
    import shutil
    if not shutil.which("nvcc") and not __import__("os").path.exists("/usr/local/cuda/bin/nvcc"):
        import pytest
        pytest.skip("the kernel library cannot be built here")
    from smolmoe_c99_b200.kernels.build import load
    lib = load()
    stages_out, parity_out = (ctypes.c_int * 64)(), (ctypes.c_int * 64)()

    def left(issued, consumed, stages):
        n = lib.sm_outstanding_fills(ctypes.c_longlong(issued), ctypes.c_longlong(consumed), stages, stages_out, parity_out)
        return [(stages_out[i], parity_out[i]) for i in range(n)]

    assert left(0, 0, 4) == [] and left(7, 7, 4) == []
    assert left(3, 0, 4) == [(0, 0), (1, 0), (2, 0)]                         # the first fills of a ring of four
    assert left(9, 6, 4) == [(2, 1), (3, 1), (0, 0)]                         # fills 6, 7, 8: second and third time round
    assert left(13, 9, 4) == [(1, 0), (2, 0), (3, 0), (0, 1)]                # a whole ring outstanding
    assert len(left(100, 3, 8)) == 8                                         # never more than the ring holds
    for issued in range(0, 40):
        for consumed in range(max(0, issued - 5), issued + 1):
            got = left(issued, consumed, 5)
            assert got == [(f % 5, (f // 5) & 1) for f in range(consumed, issued)]
