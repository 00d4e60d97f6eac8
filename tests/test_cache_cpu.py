"""Cache-manager lifecycle on CPU with a real pool of the tiny model: page allocation and table rows, prefix
adoption, window storage released behind a running request, eviction under pressure, and leak-freedom after every
request retired and the tree was emptied."""
import pytest
import torch

from minisgl.core import Req, SamplingParams
from minisgl.kvcache.pool import DSV4KVPool, PoolSizes
from minisgl.models.config import ModelConfig
from minisgl.scheduler.cache import CacheManager

PS, WINDOW = 16, 128


def _mgr(pages=32, swa=None, slots=4, max_len=1024, prefix=True):
    cfg = ModelConfig.tiny()
    pool = DSV4KVPool(cfg, PoolSizes(pages, swa if swa is not None else pages, slots, PS), "cpu")
    table = torch.zeros(slots + 1, max_len, dtype=torch.int32)
    return CacheManager(pool, table, PS, WINDOW, enable_prefix_cache=prefix), pool, table


def _req(tokens, slot=0, out=8, uid=0):
    return Req(torch.tensor(tokens, dtype=torch.int32), slot, 0, out, uid, SamplingParams())


def _prefill_done(cm, req):
    """What the scheduler does once the whole prompt went through the model."""
    cm.allocate(req, req.device_len)
    req.complete_one()
    cm.cache_req(req, finished=False)


def test_allocate_writes_token_locations_and_retire_returns_everything():
    cm, pool, table = _mgr(prefix=False)
    r = _req(list(range(40)), slot=2)
    cm.adopt_prefix(r, cm.match_req(r.input_ids))
    cm.allocate(r, 40)
    assert len(r.pages) == 3 and cm.counters["alloc_pages"] == 3
    want = torch.cat([torch.arange(p * PS, (p + 1) * PS) for p in r.pages]).to(torch.int32)
    assert torch.equal(table[2, :48], want) and int(table[2, 48:].abs().sum()) == 0
    cm.allocate(r, 48)          # already covered
    assert len(r.pages) == 3
    cm.allocate(r, 49)          # one more position -> one more page, appended after the others in the row
    assert len(r.pages) == 4 and int(table[2, 48]) == r.pages[3] * PS
    assert cm.pages_still_needed(r) == 0 and all(pool.swa_pins[p] == 1 for p in r.pages)
    cm.cache_req(r, finished=True)
    assert r.pages == [] and pool.num_free_pages == 32
    pool.assert_no_leak()


def test_second_request_adopts_the_cached_prefix_and_both_retire_cleanly():
    cm, pool, table = _mgr()
    shared = list(range(300, 300 + 160))
    a = _req(shared + [1, 2, 3], slot=0)
    cm.adopt_prefix(a, cm.match_req(a.input_ids))
    assert a.pages == [] and a.swa_pin_frontier == 0
    _prefill_done(cm, a)
    assert cm.radix.metrics["inserted_pages"] == 163 // PS
    b = _req(shared + [9, 9], slot=1, uid=1)
    m = cm.match_req(b.input_ids)
    assert m.raw_length == 160 and m.length == 128          # lcm(page, 128) boundary
    cm.adopt_prefix(b, m)
    assert b.pages == a.pages[:8] and all(pool.page_ref[p] == 3 for p in b.pages)   # a, b and the tree
    assert torch.equal(table[1, :128], table[0, :128])
    assert b.swa_pin_frontier == 0 and b.cache_handle is m.node
    b.cached_len = m.length
    _prefill_done(cm, b)
    assert len(b.pages) == 11 and b.pages[8:] != a.pages[8:11]
    assert cm.available_pages == pool.num_free_pages         # everything cached is locked by a running request
    cm.cache_req(a, finished=True)
    cm.cache_req(b, finished=True)
    snap = cm.prefix_metrics_snapshot()
    assert snap["hit_tokens"] == 128 and snap["evictable_pages"] == 32 - pool.num_free_pages > 0
    assert cm.available_pages == 32
    cm.radix.reset()
    pool.assert_no_leak()


def test_identical_prompt_leaves_at_least_one_token_for_the_model():
    cm, pool, _ = _mgr()
    toks = list(range(500, 500 + 256))
    a = _req(toks, slot=0)
    cm.adopt_prefix(a, cm.match_req(a.input_ids))
    _prefill_done(cm, a)
    cm.cache_req(a, finished=True)
    # the match runs on input_ids[:-1]: 255 tokens -> 15 whole pages -> aligned boundary 128
    m = cm.match_req(torch.tensor(toks, dtype=torch.int32))
    assert m.raw_length == 240 and m.length == 128
    # one token more and the whole cached prompt is reused
    m = cm.match_req(torch.tensor(toks + [3], dtype=torch.int32))
    assert m.raw_length == 256 and m.length == 256 and len(m.pages) == 16
    # under pressure the unpinned window rows go; a retired path keeps them only for its tail (the 128 tokens before
    # its last aligned boundary, 256): the hit at 128 backs off, the one at 256 survives
    assert pool.reclaim_swa(100) == 8
    m = cm.match_req(torch.tensor(toks, dtype=torch.int32))
    assert m.raw_length == 240 and m.length == 0 and cm.radix.metrics["swa_backoff_tokens"] >= 240
    assert cm.match_req(torch.tensor(toks + [3], dtype=torch.int32)).length == 256
    assert cm.match_req(torch.tensor(toks[:1], dtype=torch.int32)).length == 0
    cm.radix.reset()
    pool.assert_no_leak()


def test_window_storage_is_released_behind_a_running_request():
    cm, pool, _ = _mgr(prefix=False)
    r = _req(list(range(100)), out=400)
    cm.adopt_prefix(r, cm.match_req(r.input_ids))
    cm.allocate(r, 100)
    assert cm.release_swa_behind(r) == 0                     # nothing lies behind a 128-token window yet
    for n in (200, 300):
        cm.allocate(r, n)
        r.cached_len, r.device_len = n, n + 1
        cm.release_swa_behind(r)
    # positions [0, 300-128) are out of reach: 172 // 16 = 10 whole pages are unpinned; their slots can be taken
    assert r.swa_pin_frontier == 10 and r.swa_evicted_seqlen == 160 and cm.counters["swa_unpinned"] == 10
    c = pool.runtime_swa_counters()
    assert c["pages_in_use"] == 19 and c["swa_slots_reclaimable"] == 10 and c["pages_without_window"] == 0
    assert pool.num_free_swa == 32 - 19 + 10
    assert cm.release_swa_behind(r) == 0                     # idempotent
    other = _req(list(range(7000, 7100)), slot=1, uid=1, out=300)
    cm.adopt_prefix(other, cm.match_req(other.input_ids))
    cm.allocate(other, 16 * 13)                               # 13 pages: all that are free; slots: 13 unused
    assert pool.counters["swa_reclaimed"] == 0
    cm.cache_req(other, finished=True)
    pool2_need = pool.alloc_pages(13, with_swa=False)         # pages without window rows do not touch the slots
    pool.attach_swa(pool2_need)                               # 13 unused slots again, still nothing reclaimed
    assert pool.counters["swa_reclaimed"] == 0 and pool.reclaim_swa(4) == 4
    assert [pool.has_swa(p) for p in r.pages] == [False] * 4 + [True] * 15     # oldest unpinned first
    c = pool.runtime_swa_counters()
    assert c["pages_without_window"] == 4 and c["swa_slots_reclaimable"] == 6 and c["swa_reclaimed"] == 4
    pool.unref_pages(pool2_need)
    cm.cache_req(r, finished=True)
    pool.assert_no_leak()


def test_fewer_window_slots_than_pages_bound_what_a_request_can_hold():
    cm, pool, _ = _mgr(pages=32, swa=10, prefix=False)
    r = _req(list(range(64)), out=400)
    cm.adopt_prefix(r, cm.match_req(r.input_ids))
    cm.allocate(r, 160)                                      # 10 pages, 10 window slots
    with pytest.raises(RuntimeError, match="out of KV pages"):
        cm.allocate(r, 176)
    r.cached_len, r.device_len = 160, 161
    assert cm.release_swa_behind(r) == 2                     # the window moved on: two slots come back
    cm.allocate(r, 176)
    assert len(r.pages) == 11
    cm.cache_req(r, finished=True)
    pool.assert_no_leak()


def test_allocation_evicts_unlocked_prefixes_but_never_locked_ones():
    cm, pool, _ = _mgr(pages=24)
    for i in range(2):                                        # two finished prompts stay cached: 2 x 8 pages
        r = _req(list(range(1000 * (i + 1), 1000 * (i + 1) + 129)), slot=i, uid=i)
        cm.adopt_prefix(r, cm.match_req(r.input_ids))
        _prefill_done(cm, r)
        cm.cache_req(r, finished=True)
    assert pool.num_free_pages == 8 and cm.available_pages == 24
    live = _req(list(range(1000, 1000 + 129)) + [5], slot=2, uid=7)   # reuses (and locks) the first prefix
    m = cm.match_req(live.input_ids)
    cm.adopt_prefix(live, m)
    assert m.length == 128 and cm.available_pages == 16
    big = _req(list(range(5000, 5000 + 250)), slot=3, uid=8)
    cm.adopt_prefix(big, cm.match_req(big.input_ids))
    cm.allocate(big, 250)                                     # 16 pages: the 8 free ones + the unlocked cached prefix
    assert cm.counters["evictions"] == 1 and cm.radix.metrics["evicted_pages"] == 8
    assert cm.match_req(torch.tensor(list(range(2000, 2130)), dtype=torch.int32)).length == 0   # evicted
    assert cm.match_req(live.input_ids).length == 128         # the locked prefix survived
    with pytest.raises(RuntimeError, match="out of KV pages"):
        cm.allocate(big, 250 + PS)
    for r in (live, big):
        cm.cache_req(r, finished=True)
    cm.radix.reset()
    pool.assert_no_leak()


def test_row_wider_than_the_page_table_is_refused():
    cm, pool, _ = _mgr(max_len=64, prefix=False)
    r = _req(list(range(60)), out=100)
    cm.adopt_prefix(r, cm.match_req(r.input_ids))
    cm.allocate(r, 64)
    with pytest.raises(RuntimeError, match="page table width"):
        cm.allocate(r, 65)


def test_evictable_count_and_lru_are_kept_incrementally():
    """The evictable-page figure admission reads is maintained on lock / unlock / insert / evict; it must equal a
    full walk of the tree at every point, and eviction must take unlocked leaves oldest first without one."""
    cm, pool, _ = _mgr(pages=64)
    reqs = []
    for i in range(4):
        r = _req(list(range(1000 * (i + 1), 1000 * (i + 1) + 129)), slot=i % 4, uid=i)
        cm.adopt_prefix(r, cm.match_req(r.input_ids))
        _prefill_done(cm, r)
        assert cm.radix.evictable_pages() == cm.radix._count_evictable()
        reqs.append(r)
    assert cm.radix.evictable_pages() == 0                      # all four paths are locked by their requests
    for r in reqs[:3]:
        cm.cache_req(r, finished=True)
        assert cm.radix.evictable_pages() == cm.radix._count_evictable()
    assert cm.radix.evictable_pages() == 24
    cm.match_req(torch.tensor(list(range(1000, 1129)) + [1], dtype=torch.int32))   # touch the oldest path
    assert cm.radix.evict(8) == 8
    assert cm.match_req(torch.tensor(list(range(2000, 2130)), dtype=torch.int32)).length == 0   # 2nd oldest went
    assert cm.match_req(torch.tensor(list(range(1000, 1130)), dtype=torch.int32)).length == 128  # touched one stayed
    assert cm.radix.evictable_pages() == cm.radix._count_evictable() == 16
    cm.cache_req(reqs[3], finished=True)
    cm.radix.reset()
    assert cm.radix.evictable_pages() == 0
    pool.assert_no_leak()


def test_duplicate_prefix_pages_are_swapped_for_the_cached_ones():
    """Two requests prefill the same prompt at the same time; the second to finish finds its pages already in the
    tree, switches to them (page-table row included) and returns its duplicates."""
    cm, pool, table = _mgr(pages=64)
    toks = list(range(300, 300 + 161))
    a, b = _req(toks, slot=0, uid=0), _req(toks, slot=1, uid=1)
    for r in (a, b):
        cm.adopt_prefix(r, cm.match_req(r.input_ids))
        cm.allocate(r, r.device_len)
    assert not set(a.pages) & set(b.pages)
    free_before = pool.num_free_pages
    for r in (a, b):
        r.complete_one()
        cm.cache_req(r, finished=False)
    assert b.pages[:10] == a.pages[:10] and b.pages[10] != a.pages[10]      # 160 shared tokens = 10 whole pages
    assert cm.counters["dedup_pages"] == 10 and pool.num_free_pages == free_before + 10
    want = torch.cat([torch.arange(p * PS, (p + 1) * PS) for p in b.pages]).to(torch.int32)
    assert torch.equal(table[1, :len(want)], want)
    assert all(pool.swa_pins[p] >= 2 for p in a.pages[2:10])                # both requests pin the shared window pages
    for r in (a, b):
        cm.cache_req(r, finished=True)
    cm.radix.reset()
    pool.assert_no_leak()


def test_tree_gives_up_tail_pins_when_slots_run_short():
    cm, pool, _ = _mgr(pages=64, swa=20)
    a = _req(list(range(100, 100 + 161)), slot=0, uid=0, out=200)
    cm.adopt_prefix(a, cm.match_req(a.input_ids))
    _prefill_done(cm, a)                                       # 11 pages; the tree pins the tail of the locked path
    assert pool.runtime_swa_counters()["pages_pinned_by_tree"] == 8
    for n in (250, 331):                                       # decode on: the window leaves the prompt behind
        cm.allocate(a, n)
        a.cached_len, a.device_len = n - 1, n
        cm.release_swa_behind(a)
    held = pool.runtime_swa_counters()
    assert held["pages_pinned"] >= 16                           # 9 by the request, the rest by the tree
    b = _req(list(range(5000, 5000 + 150)), slot=1, uid=1)
    cm.adopt_prefix(b, cm.match_req(b.input_ids))
    assert cm.try_allocate(b, 150)                              # 10 slots: only there once the tree lets go
    assert cm.counters["tree_pins_dropped"] > 0 and cm.counters["alloc_failures"] == 0
    for r in (a, b):
        cm.cache_req(r, finished=True)
    cm.radix.reset()
    pool.assert_no_leak()
