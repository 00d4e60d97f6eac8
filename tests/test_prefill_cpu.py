"""Resident chunked prefill on CPU with the real cache manager and pool: admission against page capacity and request
slots, fair chunks across resident prompts, rotation of unfinished prompts, final-chunk marking and abort."""
import torch

from minisgl.core import SamplingParams
from minisgl.kvcache.pool import DSV4KVPool, PoolSizes
from minisgl.models.config import ModelConfig
from minisgl.scheduler.cache import CacheManager
from minisgl.scheduler.decode import DecodeManager
from minisgl.scheduler.prefill import PendingReq, PrefillManager
from minisgl.scheduler.table import TableManager

PS = 16


def _setup(pages=64, slots=4, prefix=False):
    cfg = ModelConfig.tiny()
    pool = DSV4KVPool(cfg, PoolSizes(pages, pages, slots, PS), "cpu")
    table = torch.zeros(slots + 1, 2048, dtype=torch.int32)
    cache = CacheManager(pool, table, PS, 128, enable_prefix_cache=prefix)
    tm, dm = TableManager(slots), DecodeManager(PS)
    return PrefillManager(cache, tm, dm, PS, 2048), cache, tm, dm, pool


def _pending(uid, n, out=8, base=0):
    return PendingReq(uid, torch.arange(base, base + n, dtype=torch.int32), SamplingParams(max_tokens=out))


def _ran(batch):
    """The engine's part: the granted chunk of every request went through the model."""
    for r, g in zip(batch.reqs, batch.chunk_lens):
        r.cached_len += g


def test_one_long_prompt_is_chunked_until_its_final_chunk():
    pm, cache, tm, dm, pool = _setup()
    pm.add_one_req(_pending(1, 300))
    seen = []
    while True:
        b = pm.schedule_next_batch(128)
        if b is None:
            break
        assert b.is_prefill and len(b.reqs) == 1
        seen.append((b.chunk_lens[0], b.is_final[0]))
        _ran(b)
    assert seen == [(128, False), (128, False), (44, True)]
    assert not pm.runnable and tm.available_size == 3
    assert pool.num_free_pages == 64 - 19                    # 300 prompt tokens -> 19 pages so far


def test_resident_prompts_share_the_budget_and_short_ones_finish_first():
    pm, cache, tm, dm, pool = _setup()
    pm.add_one_req(_pending(1, 400))
    pm.add_one_req(_pending(2, 40, base=1000))
    pm.add_one_req(_pending(3, 100, base=2000))
    b = pm.schedule_next_batch(128)
    by_uid = {r.uid: (g, f) for r, g, f in zip(b.reqs, b.chunk_lens, b.is_final)}
    assert sum(g for g, _ in by_uid.values()) <= 128 and set(by_uid) == {1, 2, 3}
    assert by_uid[2] == (40, True)                           # a final tail below one page is granted whole
    assert by_uid[1][0] % PS == 0 and by_uid[3][0] % PS == 0 and not by_uid[1][1]
    _ran(b)
    # the finished prompt left the resident list; the others went behind anything that did not run
    assert [r.uid for r in pm.resident] == [1, 3]
    total = {1: by_uid[1][0], 3: by_uid[3][0]}
    finals = {}
    for _ in range(10):
        b = pm.schedule_next_batch(128)
        if b is None:
            break
        for r, g, f in zip(b.reqs, b.chunk_lens, b.is_final):
            total[r.uid] += g
            if f:
                finals[r.uid] = True
        _ran(b)
    assert total == {1: 400, 3: 100} and finals == {1: True, 3: True} and not pm.resident


def test_admission_waits_for_pages_and_for_request_slots():
    pm, cache, tm, dm, pool = _setup(pages=16, slots=2)
    pm.add_one_req(_pending(1, 100, out=60))                 # 160 tokens -> 10 pages
    pm.add_one_req(_pending(2, 100, out=60, base=500))       # another 10: does not fit beside the first
    b = pm.schedule_next_batch(256)
    assert [r.uid for r in b.reqs] == [1] and len(pm.pending) == 1
    _ran(b)
    first = b.reqs[0]
    dm.add(first)                                            # it decodes now and still claims its remaining pages
    assert pm.schedule_next_batch(256) is None and len(pm.pending) == 1
    dm.remove(first)
    cache.cache_req(first, finished=True)
    tm.free(first.table_idx)
    b = pm.schedule_next_batch(256)
    assert [r.uid for r in b.reqs] == [2]
    # request slots: two short prompts take both slots, the third stays pending although pages are free
    pm2, _, tm2, _, _ = _setup(pages=64, slots=2)
    for u in (1, 2, 3):
        pm2.add_one_req(_pending(u, 20, base=100 * u))
    b = pm2.schedule_next_batch(256)
    assert [r.uid for r in b.reqs] == [1, 2] and len(pm2.pending) == 1 and tm2.available_size == 0


def test_abort_of_pending_and_resident_requests():
    pm, cache, tm, dm, pool = _setup()
    pm.add_one_req(_pending(1, 200))
    pm.add_one_req(_pending(2, 200, base=1000))
    b = pm.schedule_next_batch(64)
    _ran(b)
    pm.add_one_req(_pending(3, 50, base=2000))
    assert pm.abort(3) is None and len(pm.pending) == 0      # still queued: nothing to release
    r = pm.abort(1)
    assert r is not None and r.uid == 1 and [x.uid for x in pm.resident] == [2]
    cache.cache_req(r, finished=True)                        # the scheduler retires what abort hands back
    tm.free(r.table_idx)
    assert pm.abort(99) is None
    r2 = pm.abort(2)
    cache.cache_req(r2, finished=True)
    tm.free(r2.table_idx)
    assert not pm.runnable and tm.available_size == 4
    pool.assert_no_leak()


def test_adopted_prefix_pages_do_not_pay_for_other_requests():
    """A cached prefix counts as evictable capacity until a request adopts (and thereby locks) it.  Admission must
    not promise those pages twice: with 8 free pages, 8 cached ones and a request that already claims 8, a second
    request that would lock the cached 8 and need 8 more has to wait."""
    pm, cache, tm, dm, pool = _setup(pages=16, slots=4, prefix=True)
    pm.add_one_req(_pending(1, 129, out=1))
    b = pm.schedule_next_batch(512)
    _ran(b)
    x = b.reqs[0]
    cache.cache_req(x, finished=False)
    cache.cache_req(x, finished=True)
    tm.free(x.table_idx)
    assert pool.num_free_pages == 8 and cache.available_pages == 16
    pm.add_one_req(_pending(2, 100, out=28, base=5000))                     # 8 pages, no shared prefix
    sharer = PendingReq(3, torch.cat([torch.arange(0, 128, dtype=torch.int32), torch.tensor([7, 8], dtype=torch.int32)]),
                        SamplingParams(max_tokens=126))                     # 16 pages, 8 of them the cached prefix
    pm.add_one_req(sharer)
    b = pm.schedule_next_batch(512)
    assert [r.uid for r in b.reqs] == [2] and [p.uid for p in pm.pending] == [3]
    _ran(b)
    c = b.reqs[0]
    dm.add(c)
    assert pm.schedule_next_batch(512) is None                              # still claimed by the running request
    cache.allocate(c, c.max_device_len)                                     # it really gets its 8 pages
    dm.remove(c)
    cache.cache_req(c, finished=True)
    tm.free(c.table_idx)
    b = pm.schedule_next_batch(512)
    assert [r.uid for r in b.reqs] == [3] and b.reqs[0].cached_len == 128
    cache.allocate(b.reqs[0], b.reqs[0].max_device_len)                     # and so does the sharer: 8 adopted + 8 new
    assert len(b.reqs[0].pages) == 16
