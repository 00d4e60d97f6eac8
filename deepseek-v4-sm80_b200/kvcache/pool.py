"""Paged KV storage for the DeepSeek-V4 attention stack.

A *page* is ``page_size`` consecutive token positions of one sequence.  Its id indexes,
directly, every long-lived component the page owns:

* C4 rows    ``[page*ps/4, (page+1)*ps/4)``   of each ratio-4 layer's compressed cache (bf16 [rows,512]),
* indexer rows (same numbering) of each ratio-4 layer's FP8 key cache (u8 [rows,128] + fp32 scale [rows]),
* C128 rows  ``max(ps/128,1)`` per page of each ratio-128 layer's compressed cache,
* a 4-row checkpoint of the C4 overlap compressors (left halves of the page's last four tokens), which lets
  a prefix hit resume compression at the page boundary.

The sliding-window rows are the expensive part (every layer, every token), so they live in a
separate, much smaller pool of *SWA slots*; ``swa_map[page]`` is the slot a page currently holds
(-1 once the page has left every window and its slot was recycled).  A page therefore keeps its
compressed history for as long as the radix tree or a request references it while its window
storage is reclaimed independently -- the "independent SWA lifetime" of the reference
(python/minisgl/kvcache/deepseek_v4_pool.py:104-298, :1413-1463), here without the virtual full-token
namespace: compressed components are addressed by the page id itself.

Per-request compressor carry state (rings) is indexed by the request's table slot.
The last page id and the last table slot are reserved for the dummy request that pads CUDA-graph batches.
"""
from __future__ import annotations

from collections import OrderedDict

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..models.config import ModelConfig


@dataclass
class PoolSizes:
    num_pages: int
    num_swa_slots: int
    num_req_slots: int
    page_size: int


def bytes_per_page(cfg: ModelConfig, page_size: int) -> int:
    """Long-lived bytes one page owns across all layers (compressed rows, indexer rows, checkpoints)."""
    d, di = cfg.head_dim, cfg.index_head_dim
    n4, n128 = len(cfg.c4_layers), len(cfg.c128_layers)
    c4_rows = page_size // 4
    c128_rows = max(page_size // 128, 1)
    per = n4 * c4_rows * (d * 2 + di + 4)
    per += n4 * 4 * (2 * d + 2 * di) * 4
    per += n128 * c128_rows * d * 2
    return per + 4


def bytes_per_swa_slot(cfg: ModelConfig, page_size: int) -> int:
    return cfg.num_layers * page_size * cfg.head_dim * 2


def bytes_per_req_slot(cfg: ModelConfig) -> int:
    """Compressor ring state of one request slot."""
    d, di = cfg.head_dim, cfg.index_head_dim
    return (len(cfg.c4_layers) * 8 * (4 * d + 4 * di) + len(cfg.c128_layers) * 128 * 2 * d) * 4


class DSV4KVPool:
    def __init__(self, cfg: ModelConfig, sizes: PoolSizes, device, dtype=torch.bfloat16):
        self.cfg, self.sizes, self.device = cfg, sizes, torch.device(device)
        ps = sizes.page_size
        assert ps % 4 == 0, "page size must be a multiple of the C4 ratio"
        self.page_size = ps
        self.c4_rpp = ps // 4
        self.c128_rpp = max(ps // 128, 1)
        d, di = cfg.head_dim, cfg.index_head_dim
        n4, n128 = len(cfg.c4_layers), len(cfg.c128_layers)
        P, S, R = sizes.num_pages + 1, sizes.num_swa_slots + 1, sizes.num_req_slots + 1
        self.dummy_page, self.dummy_swa, self.dummy_slot = P - 1, S - 1, R - 1
        self.layer_c4 = {l: i for i, l in enumerate(cfg.c4_layers)}
        self.layer_c128 = {l: i for i, l in enumerate(cfg.c128_layers)}
        z = dict(device=self.device)
        self.swa = torch.zeros(cfg.num_layers, S * ps, d, dtype=dtype, **z)
        self.c4 = torch.zeros(max(n4, 1), P * self.c4_rpp, d, dtype=dtype, **z)
        self.c128 = torch.zeros(max(n128, 1), P * self.c128_rpp, d, dtype=dtype, **z)
        self.idx_vals = torch.zeros(max(n4, 1), P * self.c4_rpp, di, dtype=torch.uint8, **z)
        self.idx_scale = torch.zeros(max(n4, 1), P * self.c4_rpp, dtype=torch.float32, **z)
        self.c4_ring = torch.zeros(max(n4, 1), R * 8, 4 * d, dtype=torch.float32, **z)
        self.idx_ring = torch.zeros(max(n4, 1), R * 8, 4 * di, dtype=torch.float32, **z)
        self.c128_ring = torch.zeros(max(n128, 1), R * 128, 2 * d, dtype=torch.float32, **z)
        self.c4_ckpt = torch.zeros(max(n4, 1), P * 4, 2 * d, dtype=torch.float32, **z)
        self.idx_ckpt = torch.zeros(max(n4, 1), P * 4, 2 * di, dtype=torch.float32, **z)
        self.swa_map = torch.full((P,), -1, dtype=torch.int32, **z)
        self.swa_map[self.dummy_page] = self.dummy_swa
        # host-side ownership
        self._swa_map_host = [-1] * P
        self._swa_map_host[self.dummy_page] = self.dummy_swa
        self.free_pages: List[int] = list(range(sizes.num_pages - 1, -1, -1))
        self.free_swa: List[int] = list(range(sizes.num_swa_slots - 1, -1, -1))
        self.page_ref = [0] * P
        self.swa_pins = [0] * P          # users of a page's window storage (running requests + the radix tree)
        self._tree_pinned: "OrderedDict[int, None]" = OrderedDict()   # pages the prefix tree pins, oldest pin first
        self.swa_version = 0
        # pages nobody pins any more but that still own a window slot, oldest first: their rows stay readable (a later
        # prefix hit can resume on them) until another page needs the slot
        self._reclaimable: "OrderedDict[int, None]" = OrderedDict()
        self.counters = {"swa_taken": 0, "swa_released": 0, "swa_reclaimed": 0, "pages_taken": 0, "pages_released": 0}

    # ------------------------------------------------------------------ pages
    @property
    def num_free_pages(self) -> int:
        return len(self.free_pages)

    @property
    def num_free_swa(self) -> int:
        """Window slots a new page can get: unused ones plus those of unpinned pages (reclaimed on demand)."""
        return len(self.free_swa) + len(self._reclaimable)

    def alloc_pages(self, n: int, with_swa: bool = True) -> List[int]:
        if n > len(self.free_pages) or (with_swa and n > self.num_free_swa):
            raise RuntimeError(f"KV pool exhausted: want {n} pages, free {len(self.free_pages)} pages / "
                               f"{self.num_free_swa} SWA slots")
        pages = [self.free_pages.pop() for _ in range(n)]
        for p in pages:
            assert self.page_ref[p] == 0, f"page {p} handed out while referenced"
            self.page_ref[p] = 1
        self.counters["pages_taken"] += n
        if with_swa:
            self.attach_swa(pages)
        return pages

    def ref_pages(self, pages) -> None:
        for p in pages:
            assert self.page_ref[p] > 0, f"page {p} referenced while free"
            self.page_ref[p] += 1

    def unref_pages(self, pages) -> None:
        """Drops one reference; a page whose count reaches zero returns to the free list with its SWA slot."""
        freed = []
        for p in pages:
            assert self.page_ref[p] > 0, f"double free of page {p}"
            self.page_ref[p] -= 1
            if self.page_ref[p] == 0:
                freed.append(p)
        if freed:
            for p in freed:
                self.swa_pins[p] = 0
                self._tree_pinned.pop(p, None)
            self.release_swa(freed)
            self.free_pages.extend(freed)
            self.counters["pages_released"] += len(freed)

    # ------------------------------------------------------------------ SWA slots
    def reclaim_swa(self, n: int) -> int:
        """Takes the window slots of up to n unpinned pages back, least recently unpinned first."""
        victims = []
        while len(victims) < n and self._reclaimable:
            victims.append(self._reclaimable.popitem(last=False)[0])
        if victims:
            self.counters["swa_reclaimed"] += len(victims)
            self.release_swa(victims)
        return len(victims)

    def attach_swa(self, pages) -> None:
        need = sum(1 for p in pages if self._swa_map_host[p] < 0)
        if need > len(self.free_swa):
            self.reclaim_swa(need - len(self.free_swa))
        upd_p, upd_s = [], []
        for p in pages:
            if self._swa_map_host[p] >= 0:
                continue
            if not self.free_swa:
                raise RuntimeError("SWA pool exhausted")
            s = self.free_swa.pop()
            self._swa_map_host[p] = s
            upd_p.append(p)
            upd_s.append(s)
        if upd_p:
            self.counters["swa_taken"] += len(upd_p)
            self._push_swa_map(upd_p, upd_s)

    def release_swa(self, pages) -> int:
        """Recycles the SWA slots of pages that left every window (tombstoning); the pages stay valid."""
        upd = []
        for p in pages:
            s = self._swa_map_host[p]
            self._reclaimable.pop(p, None)
            if s >= 0 and p != self.dummy_page:
                self.free_swa.append(s)
                self._swa_map_host[p] = -1
                upd.append(p)
        if upd:
            self.counters["swa_released"] += len(upd)
            self._push_swa_map(upd, [-1] * len(upd))
        return len(upd)

    def pin_swa(self, pages, owner: str = "req") -> None:
        """Declares a user of the pages' window storage.  The tree pins a page at most once."""
        for p in pages:
            if owner == "tree":
                if p in self._tree_pinned:
                    continue
                self._tree_pinned[p] = None
            self.swa_pins[p] += 1
            self._reclaimable.pop(p, None)

    def unpin_swa(self, pages, owner: str = "req") -> None:
        """Drops a user.  A page nobody pins any more keeps its window rows for as long as no other page needs the
        slot (it becomes reclaimable), so that a prefix hit ending on it can still resume there."""
        drop = []
        for p in pages:
            if owner == "tree":
                if p not in self._tree_pinned:
                    continue
                del self._tree_pinned[p]
            if self.swa_pins[p] > 0:
                self.swa_pins[p] -= 1
                if self.swa_pins[p] == 0:
                    drop.append(p)
        for p in drop:
            if self._swa_map_host[p] >= 0 and p != self.dummy_page:
                self._reclaimable[p] = None
                self._reclaimable.move_to_end(p)

    def drop_tree_pins(self, n_slots: int) -> int:
        """Makes the prefix tree give up pins, oldest first, until n_slots more window slots are obtainable (or no
        tree pin is left).  Only pages that nobody else pins yield a slot.  The pages stay cached; a later prefix hit
        that would resume on them backs off to an earlier boundary.  Returns the number of pins dropped."""
        got = dropped = 0
        for p in list(self._tree_pinned):
            if got >= n_slots:
                break
            before = self.num_free_swa
            self.unpin_swa([p], "tree")
            dropped += 1
            got += self.num_free_swa - before
        self.counters["tree_pins_dropped"] = self.counters.get("tree_pins_dropped", 0) + dropped
        return dropped

    def runtime_swa_counters(self) -> dict:
        """Window-storage residency at this moment plus the lifetime counters: slots in use / free, pages whose
        window rows were recycled while the page stayed valid (tombstoned), pins by owner, and how often the device
        copy of the page -> slot map changed (python/minisgl/kvcache/deepseek_v4_pool.py:1206-1227 of the reference
        reports the same residency figures)."""
        live = sum(1 for p, s in enumerate(self._swa_map_host) if s >= 0 and p != self.dummy_page)
        held = sum(1 for p in range(self.sizes.num_pages) if self.page_ref[p] > 0)
        return {
            "swa_slots_total": self.sizes.num_swa_slots,
            "swa_slots_in_use": live,
            "swa_slots_free": len(self.free_swa),
            "swa_slots_reclaimable": len(self._reclaimable),
            "pages_in_use": held,
            "pages_without_window": held - sum(1 for p in range(self.sizes.num_pages)
                                               if self.page_ref[p] > 0 and self._swa_map_host[p] >= 0),
            "pages_pinned_by_tree": len(self._tree_pinned),
            "pages_pinned": sum(1 for c in self.swa_pins if c > 0),
            "swa_map_version": self.swa_version,
            **self.counters,
        }

    def has_swa(self, page: int) -> bool:
        return self._swa_map_host[page] >= 0

    def swa_slot(self, page: int) -> int:
        return self._swa_map_host[page]

    def _push_swa_map(self, pages, slots) -> None:
        self.swa_version += 1
        idx = torch.tensor(pages, dtype=torch.int64)
        val = torch.tensor(slots, dtype=torch.int32)
        if self.device.type == "cuda":
            idx = idx.pin_memory().to(self.device, non_blocking=True)
            val = val.pin_memory().to(self.device, non_blocking=True)
        self.swa_map[idx] = val

    # ------------------------------------------------------------------ views
    def layer_views(self, layer: int) -> dict:
        r = self.cfg.ratio(layer)
        v = {"swa": self.swa[layer], "ratio": r}
        if r == 4:
            i = self.layer_c4[layer]
            v.update(comp=self.c4[i], ring=self.c4_ring[i], ckpt=self.c4_ckpt[i], idx_vals=self.idx_vals[i],
                     idx_scale=self.idx_scale[i], idx_ring=self.idx_ring[i], idx_ckpt=self.idx_ckpt[i])
        elif r:
            i = self.layer_c128[layer]
            v.update(comp=self.c128[i], ring=self.c128_ring[i], ckpt=None)
        return v

    def assert_no_leak(self) -> None:
        assert len(self.free_pages) == self.sizes.num_pages, (len(self.free_pages), self.sizes.num_pages)
        assert len(self.free_swa) == self.sizes.num_swa_slots, (len(self.free_swa), self.sizes.num_swa_slots)
        assert all(r == 0 for r in self.page_ref[:-1])
        assert all(s == -1 for s in self._swa_map_host[:-1])
