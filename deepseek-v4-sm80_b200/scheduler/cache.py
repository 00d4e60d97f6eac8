"""Page bookkeeping for running requests: prefix matching, page allocation with eviction, page-table rows,
radix insertion, and the independent release of sliding-window storage behind each request's window.

Ownership rules (compare python/minisgl/scheduler/cache.py:55-531 of the reference, whose virtual full-token
namespace this design does not need):
  * a request holds one pool reference on every page in ``req.pages`` (matched prefix pages included) and drops
    them all when it retires; the radix tree holds its own reference on every page it stores;
  * a request *pins* the window storage of the pages its sliding window can still reach and unpins pages as the
    window moves past them (``release_swa_behind``); the tree pins the tail of each cached path;
  * pages are inserted into the tree when a prompt finishes prefill and again when the request retires (whole
    pages of tokens that went through the model).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..core import Req
from ..kvcache.radix_cache import MatchResult, RadixPrefixCache
from ..utils.misc import div_ceil


class KVExhausted(RuntimeError):
    """No page (or no sliding-window slot) could be freed for an allocation.  The scheduler never lets it escape its
    loop: a prefill chunk that cannot get storage is deferred, a decoding request that cannot is ended."""


def slots_per_request(window: int, page_size: int) -> int:
    """Window slots one admitted request can need at the same time outside a prefill chunk: the pages its window
    reaches (``ceil(window / ps)`` plus the page being written) and one more for the step that overlap scheduling
    keeps in flight.  Slots pinned by the prefix tree are not part of it: under pressure the tree gives them up
    (``DSV4KVPool.drop_tree_pins``), which only costs later prefix hits their resume point."""
    return div_ceil(window, page_size) + 2


class CacheManager:
    def __init__(self, pool, page_table: torch.Tensor, page_size: int, window: int, enable_prefix_cache: bool = True):
        self.pool, self.page_table, self.ps, self.window = pool, page_table, page_size, window
        self.radix: Optional[RadixPrefixCache] = RadixPrefixCache(pool, page_size, window) if enable_prefix_cache else None
        self.device = page_table.device
        self.counters = {"alloc_pages": 0, "evictions": 0, "swa_unpinned": 0, "alloc_failures": 0, "dedup_pages": 0,
                         "tree_pins_dropped": 0}

    # ------------------------------------------------------------------ capacity
    @property
    def available_pages(self) -> int:
        ev = self.radix.evictable_pages() if self.radix else 0
        return self.pool.num_free_pages + ev

    def pages_still_needed(self, req: Req) -> int:
        return max(div_ceil(req.max_device_len, self.ps) - len(req.pages), 0)

    def request_capacity(self, prefill_budget: int) -> int:
        """How many requests the window-slot pool can carry at once: what is left of the pool after one prefill
        forward's pages (at most half of it) and a spare, divided by each request's share; never less than one (a
        lone request always fits: its chunk shrinks to what the pool can hold)."""
        total = self.pool.sizes.num_swa_slots
        chunk = min(div_ceil(prefill_budget, self.ps) + 1, total // 2)
        return max((total - chunk) // slots_per_request(self.window, self.ps), 1)

    def _ensure(self, n: int) -> bool:
        """Frees storage until n pages AND n window slots are available: evicts unlocked cached paths oldest first (a
        path's pages and the slots its tail pins come back together), then, for slots only, makes the prefix tree give
        up tail pins of paths that running requests keep locked.  Returns whether it succeeded."""
        pool = self.pool
        evicted = False
        while (pool.num_free_pages < n or pool.num_free_swa < n) and self.radix is not None:
            if self.radix.evict(max(n - pool.num_free_pages, 1)) == 0:
                break
            evicted = True
        if evicted:
            self.counters["evictions"] += 1
        if pool.num_free_swa < n:
            self.counters["tree_pins_dropped"] += pool.drop_tree_pins(n - pool.num_free_swa)
        return pool.num_free_pages >= n and pool.num_free_swa >= n

    # ------------------------------------------------------------------ prefix reuse
    def match_req(self, input_ids: torch.Tensor) -> MatchResult:
        """Prefix match on input_ids[:-1]: at least one token must still go through the model."""
        if self.radix is None or len(input_ids) <= 1:
            return MatchResult(0, [], None, 0)
        return self.radix.match(input_ids[:-1].numpy())

    def adopt_prefix(self, req: Req, m: MatchResult) -> None:
        """Takes references on the matched pages, pins the window tail, locks the tree path, fills the table row."""
        if m.length == 0:
            req.swa_pin_frontier = 0
            return
        self.pool.ref_pages(m.pages)
        req.pages = list(m.pages)
        first = max(m.length - self.window, 0) // self.ps
        self.pool.pin_swa(m.pages[first:], "req")
        req.swa_pin_frontier = first
        self.radix.lock(m.node)
        req.cache_handle = m.node
        self._write_rows(req.table_idx, 0, m.pages)

    # ------------------------------------------------------------------ allocation
    def try_allocate(self, req: Req, upto_len: int) -> bool:
        """``allocate`` that reports exhaustion instead of raising (nothing is allocated then)."""
        try:
            self.allocate(req, upto_len)
            return True
        except KVExhausted:
            self.counters["alloc_failures"] += 1
            return False

    def allocate(self, req: Req, upto_len: int) -> None:
        """Makes req.pages cover positions [0, upto_len); raises :class:`KVExhausted` (and allocates nothing) when
        neither free storage nor eviction can supply the pages and their window slots."""
        need = div_ceil(upto_len, self.ps) - len(req.pages)
        if need <= 0:
            return
        if (len(req.pages) + need) * self.ps > self.page_table.shape[1]:
            raise RuntimeError("request exceeds the page table width (max sequence length)")
        if not self._ensure(need):
            raise KVExhausted(f"out of KV pages: need {need}, free pages {self.pool.num_free_pages}, "
                              f"free SWA slots {self.pool.num_free_swa}")
        new = self.pool.alloc_pages(need)
        self.pool.pin_swa(new, "req")
        self.counters["alloc_pages"] += need
        start = len(req.pages)
        req.pages.extend(new)
        self._write_rows(req.table_idx, start, new)

    def _write_rows(self, slot: int, first_page_index: int, pages: List[int]) -> None:
        ps = self.ps
        locs = (np.asarray(pages, dtype=np.int64)[:, None] * ps + np.arange(ps, dtype=np.int64)[None, :]).ravel()
        t = torch.from_numpy(locs.astype(np.int32))
        a = first_page_index * ps
        if a + len(t) > self.page_table.shape[1]:
            raise RuntimeError("request exceeds the page table width (max sequence length)")
        if self.device.type == "cuda":
            t = t.pin_memory().to(self.device, non_blocking=True)
        self.page_table[slot, a:a + len(t)] = t

    # ------------------------------------------------------------------ window storage
    def release_swa_behind(self, req: Req) -> int:
        """Unpins pages that lie wholly behind the window of every position the request still has to run; returns
        how many.  The next forward of the request starts at ``cached_len`` (the next prefill chunk, or the next decode
        token), whose window reaches back to ``cached_len - window + 1``.  ``device_len`` must not be used here:
        while a prompt is prefilled in chunks it already is the full prompt length."""
        target = max(req.cached_len - self.window, 0) // self.ps
        target = min(target, len(req.pages))
        frontier = getattr(req, "swa_pin_frontier", 0)
        if target <= frontier:
            return 0
        self.pool.unpin_swa(req.pages[frontier:target], "req")
        req.swa_pin_frontier = target
        req.swa_evicted_seqlen = target * self.ps
        self.counters["swa_unpinned"] += target - frontier
        return target - frontier

    # ------------------------------------------------------------------ caching / retirement
    def cache_req(self, req: Req, finished: bool) -> None:
        """Publishes the request's whole, model-visited pages to the prefix tree; on ``finished`` also returns every
        page reference, window pin and tree lock the request holds."""
        if self.radix is not None:
            valid = min(req.cached_len, len(req.input_ids))
            n = valid // self.ps * self.ps
            if n > 0:
                canon, node = self.radix.insert(req.input_ids[:n].numpy(), req.pages[: n // self.ps])
                self.radix.lock(node)
                self.radix.unlock(req.cache_handle)
                req.cache_handle = node
                if not finished:
                    self._adopt_canonical(req, canon)
        if finished:
            frontier = getattr(req, "swa_pin_frontier", 0)
            self.pool.unpin_swa(req.pages[frontier:], "req")
            if self.radix is not None:
                self.radix.unlock(req.cache_handle)
            req.cache_handle = None
            self.pool.unref_pages(req.pages)
            req.pages = []
            req.swa_pin_frontier = 0

    def _adopt_canonical(self, req: Req, canon: List[int]) -> None:
        """Where the tree already held a page for the same tokens (another request cached the same prefix first), the
        request switches to the tree's page and gives its duplicate back, as the reference does when it repoints a
        request to canonical prefix pages (python/minisgl/scheduler/cache.py:140-229).  A page that the request's
        window still reaches is only switched if the tree's page still owns window rows; the pin moves with it."""
        frontier = getattr(req, "swa_pin_frontier", 0)
        for i, c in enumerate(canon):
            own = req.pages[i]
            if c == own:
                continue
            pinned = i >= frontier
            if pinned and not self.pool.has_swa(c):
                continue
            self.pool.ref_pages([c])
            if pinned:
                self.pool.pin_swa([c], "req")
                self.pool.unpin_swa([own], "req")
            req.pages[i] = c
            self.pool.unref_pages([own])
            self._write_rows(req.table_idx, i, [c])
            self.counters["dedup_pages"] += 1

    def assert_window_resident(self, req: Req, first_pos: int, last_pos: int) -> None:
        """Invariant of every forward: each page that the sliding windows of positions [first_pos, last_pos] reach
        still owns window storage and is pinned by somebody.  Checked by the scheduler before each launch when
        ``check_window`` is set (tests, MINISGL_DEBUG_BOUNDS=1)."""
        lo = max(first_pos - self.window + 1, 0) // self.ps
        hi = last_pos // self.ps
        for i in range(lo, hi + 1):
            p = req.pages[i]
            if not self.pool.has_swa(p) or self.pool.swa_pins[p] <= 0:
                raise AssertionError(
                    f"request {req.uid}: page index {i} (page {p}) is inside the window of positions "
                    f"[{first_pos}, {last_pos}] but has_swa={self.pool.has_swa(p)} pins={self.pool.swa_pins[p]}")

    def prefix_metrics_snapshot(self) -> dict:
        m = self.radix.snapshot() if self.radix else {}
        m.update(self.counters)
        m.update({"free_pages": self.pool.num_free_pages, "free_swa_slots": self.pool.num_free_swa,
                  **{f"pool_{k}": v for k, v in self.pool.counters.items()}})
        return m

    def check_integrity(self) -> None:
        assert self.pool.num_free_pages <= self.pool.sizes.num_pages
        assert self.pool.num_free_swa <= self.pool.sizes.num_swa_slots
