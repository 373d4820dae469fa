"""Page pool, slot pool and the prefix / session-tail cache on their own (no model)."""

import pytest

from b200serve.cache.pools import OutOfCapacity, PagePool, SlotPool
from b200serve.cache.prefix import PrefixCache

BLOCK = 64


def _cache(pages=64, slots=8, **kw):
    box = []
    pp = PagePool(pages, on_pressure=lambda: box[0].evict_one())
    sp = SlotPool(slots, on_pressure=lambda: box[0].evict_one())
    c = PrefixCache(pp, sp, page_bytes=1000, slot_bytes=5000, **kw)
    box.append(c)
    return pp, sp, c


def test_pools_hand_out_low_ids_keep_page_zero_and_refuse_when_empty():
    pp = PagePool(5)
    assert pp.alloc(2) == [1, 2] and pp.free == 2 and pp.used == 2
    pp.incref([1])
    pp.release([1, 2])
    assert pp.refcount(1) == 1 and pp.refcount(2) == 0 and pp.free == 3
    with pytest.raises(OutOfCapacity):
        pp.alloc(4)
    sp = SlotPool(3)
    assert {sp.alloc(), sp.alloc()} == {1, 2}
    with pytest.raises(OutOfCapacity):
        sp.alloc()
    sp.release(1)
    assert sp.alloc() == 1


def test_a_tail_is_handed_over_once_and_only_to_a_longer_prompt():
    pp, sp, c = _cache()
    toks = list(range(100, 250))  # 150 tokens: 2 full blocks + 22
    pages, slot = pp.alloc(3), sp.alloc()
    c.store_tail(toks, pages, slot)
    assert len(c) == 1 and c.tokens == 150
    assert c.lookup(toks) is None  # needs at least one row left to compute
    assert c.lookup(toks[:149] + [7]) is None  # diverges inside the tail
    e = c.lookup(toks + [1, 2, 3])
    assert e is not None and e.kind == "tail" and e.length == 150 and e.pages == pages and e.slot == slot
    assert len(c) == 0 and c.lookup(toks + [1, 2, 3]) is None  # ownership moved to the caller
    assert c.stats.tail_hits == 1 and pp.used == 3  # the caller now owns pages and slot


def test_snapshots_share_pages_by_reference_and_serve_diverging_prompts():
    pp, sp, c = _cache()
    toks = list(range(300))
    pages = pp.alloc(5)
    assert c.store_snapshot(toks, 128, pages, sp.alloc()) is True
    assert c.store_snapshot(toks, 128, pages, 99) is False  # already there: nothing taken
    assert [pp.refcount(p) for p in pages] == [2, 2, 1, 1, 1] and c.has_snapshot(toks, 128)
    e = c.lookup(toks[:200] + [9, 9, 9])
    assert e.kind == "snapshot" and e.length == 128 and len(c) == 1  # a snapshot stays in the cache
    assert c.lookup(toks[:100] + [5] * 50) is None  # differs inside the snapshot's blocks
    pp.release(pages)  # the request that made it goes away: the shared pages live on
    assert [pp.refcount(p) for p in pages[:2]] == [1, 1] and pp.used == 2
    c.clear()
    assert pp.used == 0 and sp.free == 7 and c.tokens == 0 and c.bytes == 0


def test_the_longest_usable_entry_wins():
    pp, sp, c = _cache()
    toks = list(range(400))
    c.store_snapshot(toks, 64, pp.alloc(1), sp.alloc())
    c.store_snapshot(toks, 192, pp.alloc(3), sp.alloc())
    c.store_tail(toks[:230], pp.alloc(4), sp.alloc())
    assert c.lookup(toks[:200]).length == 192
    assert c.lookup(toks[:150]).length == 64
    assert c.lookup(toks[:300]).kind == "tail"


def test_budgets_evict_least_recently_used_first():
    pp, sp, c = _cache(max_entries=3)
    prompts = [[i] * 64 + list(range(70)) for i in range(1, 5)]
    for p in prompts[:3]:
        c.store_snapshot(p, 64, pp.alloc(1), sp.alloc())
    assert c.lookup(prompts[0]) is not None  # touch the oldest: it becomes the most recent
    c.store_snapshot(prompts[3], 64, pp.alloc(1), sp.alloc())
    assert len(c) == 3 and c.stats.evictions == 1
    assert c.lookup(prompts[1]) is None and c.lookup(prompts[0]) is not None and c.lookup(prompts[2]) is not None
    pp2, sp2, byt = _cache(max_bytes=12000)  # two state copies of 5000 bytes fit, three do not
    for p in prompts[:3]:
        byt.store_snapshot(p, 64, pp2.alloc(1), sp2.alloc())
    assert len(byt) == 2 and byt.bytes == 10000
    pp3, sp3, tok = _cache(max_tokens=200)
    tok.store_tail(list(range(150)), pp3.alloc(3), sp3.alloc())
    tok.store_tail(list(range(1000, 1100)), pp3.alloc(2), sp3.alloc())
    assert len(tok) == 1 and tok.tokens == 100 and pp3.used == 2


def test_pressure_on_pages_or_slots_evicts_cached_entries():
    pp, sp, c = _cache(pages=9, slots=4)
    c.store_tail(list(range(200)), pp.alloc(4), sp.alloc())
    c.store_tail(list(range(500, 700)), pp.alloc(4), sp.alloc())
    assert pp.free == 0
    got = pp.alloc(6)  # both tails have to go
    assert len(got) == 6 and len(c) == 0 and c.stats.evictions == 2
    pp.release(got)
    c.store_tail(list(range(70)), pp.alloc(2), sp.alloc())
    while sp.free:
        sp.alloc()
    assert len(c) == 1
    sp.alloc()  # a parked tail never blocks a request: it is evicted for its slot
    assert len(c) == 0
    with pytest.raises(OutOfCapacity):
        sp.alloc()
