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


class CacheManager:
    def __init__(self, pool, page_table: torch.Tensor, page_size: int, window: int, enable_prefix_cache: bool = True):
        self.pool, self.page_table, self.ps, self.window = pool, page_table, page_size, window
        self.radix: Optional[RadixPrefixCache] = RadixPrefixCache(pool, page_size, window) if enable_prefix_cache else None
        self.device = page_table.device
        self.counters = {"alloc_pages": 0, "evictions": 0, "swa_unpinned": 0}

    # ------------------------------------------------------------------ capacity
    @property
    def available_pages(self) -> int:
        ev = self.radix.evictable_pages() if self.radix else 0
        return self.pool.num_free_pages + ev

    def pages_still_needed(self, req: Req) -> int:
        return max(div_ceil(req.max_device_len, self.ps) - len(req.pages), 0)

    def _ensure(self, n: int) -> None:
        short = max(n - self.pool.num_free_pages, n - self.pool.num_free_swa, 0)
        if short > 0 and self.radix is not None:
            self.counters["evictions"] += 1
            self.radix.evict(short)
        if n > self.pool.num_free_pages or n > self.pool.num_free_swa:
            raise RuntimeError(f"out of KV pages: need {n}, free pages {self.pool.num_free_pages}, "
                               f"free SWA slots {self.pool.num_free_swa}")

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
    def allocate(self, req: Req, upto_len: int) -> None:
        """Makes req.pages cover positions [0, upto_len)."""
        need = div_ceil(upto_len, self.ps) - len(req.pages)
        if need <= 0:
            return
        self._ensure(need)
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
        """Unpins pages that lie wholly behind the request's sliding window; returns how many."""
        target = max(req.device_len - self.window, 0) // self.ps
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
                _, node = self.radix.insert(req.input_ids[:n].numpy(), req.pages[: n // self.ps])
                self.radix.lock(node)
                self.radix.unlock(req.cache_handle)
                req.cache_handle = node
        if finished:
            frontier = getattr(req, "swa_pin_frontier", 0)
            self.pool.unpin_swa(req.pages[frontier:], "req")
            if self.radix is not None:
                self.radix.unlock(req.cache_handle)
            req.cache_handle = None
            self.pool.unref_pages(req.pages)
            req.pages = []
            req.swa_pin_frontier = 0

    def prefix_metrics_snapshot(self) -> dict:
        m = self.radix.snapshot() if self.radix else {}
        m.update(self.counters)
        m.update({"free_pages": self.pool.num_free_pages, "free_swa_slots": self.pool.num_free_swa,
                  **{f"pool_{k}": v for k, v in self.pool.counters.items()}})
        return m

    def check_integrity(self) -> None:
        assert self.pool.num_free_pages <= self.pool.sizes.num_pages
        assert self.pool.num_free_swa <= self.pool.sizes.num_swa_slots
