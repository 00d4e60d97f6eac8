"""Page-granular radix tree over token ids: the prefix cache.

A node owns a run of whole pages: ``tokens`` (int32, a multiple of ``page_size`` long) and the page ids that
hold them.  The tree holds one pool reference per page it stores.  Requests *lock* the path they reuse
(``lock``/``unlock`` bump a per-node counter) so that eviction, which removes least-recently-used unlocked
leaves, never frees pages under a running request.  Node runs are compared with the native
``dsv4_first_mismatch`` (the reference does the same comparison in C++: python/minisgl/kernel/csrc/src/radix.cpp:19-44;
its tree is python/minisgl/kvcache/radix_cache.py:165-620).

Sliding-window storage has its own lifetime: a cached page keeps its SWA slot only while it is the *tail* of a
cached path (so that a later prefix hit can resume right after it) or while a running request's window still
covers it.  ``match`` therefore backs a hit off to the longest boundary whose preceding ``window`` tokens still
have window storage, and to a multiple of ``align`` tokens (128 for the ratio-128 compressor, whose ring holds
no partial group at such boundaries).
"""
from __future__ import annotations

import heapq
import itertools
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..ops import native


def first_mismatch(a: np.ndarray, b: np.ndarray) -> int:
    n = min(len(a), len(b))
    if n == 0:
        return 0
    a = np.ascontiguousarray(a[:n], dtype=np.int32)
    b = np.ascontiguousarray(b[:n], dtype=np.int32)
    try:
        lib = native.host_lib()
        return int(lib.dsv4_first_mismatch(a.ctypes.data, b.ctypes.data, n, 4))
    except OSError:
        neq = np.nonzero(a != b)[0]
        return int(neq[0]) if len(neq) else n


class RadixNode:
    _ids = itertools.count()

    def __init__(self, tokens: np.ndarray, pages: List[int], parent: Optional["RadixNode"]):
        self.tokens, self.pages, self.parent = tokens, pages, parent
        self.children: Dict[bytes, RadixNode] = {}
        self.lock_count = 0
        self.last_access = time.monotonic()
        self.uid = next(RadixNode._ids)

    @property
    def is_leaf(self) -> bool:
        return not self.children

    def path_len(self) -> int:
        n, node = 0, self
        while node is not None:
            n += len(node.tokens)
            node = node.parent
        return n


@dataclass
class MatchResult:
    length: int                 # reusable tokens (page aligned, possibly backed off)
    pages: List[int]            # their page ids, in order
    node: Optional[RadixNode]   # deepest node of the reused path (lock this)
    raw_length: int = 0         # what the tree had before the window / alignment back-off


class RadixPrefixCache:
    def __init__(self, pool, page_size: int, window: int, align: int = 128):
        self.pool, self.ps, self.window = pool, page_size, window
        self.align = int(np.lcm(align, page_size))
        self.root = RadixNode(np.zeros(0, np.int32), [], None)
        self.root.lock_count = 1
        # kept incrementally, so that admission checks and eviction never walk the tree: pages held by unlocked
        # nodes, and a lazily cleaned heap of (last_access, uid, node) candidates (an entry is stale when its node
        # left the tree, got children, got locked or was touched since)
        self._evictable = 0
        self._lru: list = []
        self._nodes = 0
        self.metrics = {"queries": 0, "hit_tokens": 0, "query_tokens": 0, "evicted_pages": 0, "inserted_pages": 0,
                        "swa_backoff_tokens": 0}

    # ------------------------------------------------------------------ helpers
    def _key(self, tokens: np.ndarray) -> bytes:
        return tokens[: self.ps].tobytes()

    def _split(self, node: RadixNode, n_tokens: int) -> RadixNode:
        """Splits ``node`` after n_tokens (page aligned); returns the new upper node."""
        npg = n_tokens // self.ps
        upper = RadixNode(node.tokens[:n_tokens], node.pages[:npg], node.parent)
        upper.lock_count = node.lock_count
        upper.last_access = node.last_access
        self._nodes += 1
        node.parent.children[self._key(node.tokens)] = upper
        node.tokens, node.pages, node.parent = node.tokens[n_tokens:], node.pages[npg:], upper
        upper.children[self._key(node.tokens)] = node
        return upper

    def _walk(self, tokens: np.ndarray, split: bool) -> Tuple[RadixNode, int]:
        node, done = self.root, 0
        now = time.monotonic()
        while len(tokens) - done >= self.ps:
            child = node.children.get(self._key(tokens[done:]))
            if child is None:
                break
            n = first_mismatch(child.tokens, tokens[done:]) // self.ps * self.ps
            if n == 0:
                break
            child.last_access = now
            self._offer(child)
            if n < len(child.tokens):
                if not split:
                    return child, done + n  # partial use of the child's run
                child = self._split(child, n)
            node, done = child, done + n
            if n < len(child.tokens):
                break
        return node, done

    def _path_pages(self, node: RadixNode, length: int) -> List[int]:
        chain = []
        while node is not None and node is not self.root:
            chain.append(node)
            node = node.parent
        pages: List[int] = []
        for nd in reversed(chain):
            pages.extend(nd.pages)
        return pages[: length // self.ps]

    # ------------------------------------------------------------------ API
    def match(self, tokens) -> MatchResult:
        """Longest reusable prefix of ``tokens`` (callers pass input_ids[:-1])."""
        tokens = np.asarray(tokens, dtype=np.int32)
        self.metrics["queries"] += 1
        self.metrics["query_tokens"] += len(tokens)
        node, raw = self._walk(tokens, split=True)
        pages = self._path_pages(node, raw)
        length = raw // self.align * self.align
        # back off until the window before the boundary still has sliding-window storage
        while length > 0:
            first = max(length - self.window, 0) // self.ps
            if all(self.pool.has_swa(p) for p in pages[first: length // self.ps]):
                break
            length -= self.align
        length = max(length, 0)
        self.metrics["swa_backoff_tokens"] += raw - length
        self.metrics["hit_tokens"] += length
        if length < raw:
            node, _ = self._walk(tokens[:length], split=True) if length else (self.root, 0)
        return MatchResult(length, pages[: length // self.ps], node if length else None, raw)

    def _offer(self, node: RadixNode) -> None:
        """Registers ``node`` as an eviction candidate if it is one right now."""
        if node is not self.root and node.lock_count == 0 and node.is_leaf and node.parent is not None:
            heapq.heappush(self._lru, (node.last_access, node.uid, node))
            if len(self._lru) > 64 + 8 * self._nodes:   # drop stale entries
                live = {}
                for t, u, nd in self._lru:
                    if nd.parent is not None and nd.lock_count == 0 and nd.is_leaf and t == nd.last_access:
                        live[u] = (t, u, nd)
                self._lru = list(live.values())
                heapq.heapify(self._lru)

    def lock(self, node: Optional[RadixNode]) -> None:
        while node is not None and node is not self.root:
            if node.lock_count == 0:
                self._evictable -= len(node.pages)
            node.lock_count += 1
            node = node.parent

    def unlock(self, node: Optional[RadixNode]) -> None:
        while node is not None and node is not self.root:
            assert node.lock_count > 0, "unlock of an unlocked radix node"
            node.lock_count -= 1
            if node.lock_count == 0:
                self._evictable += len(node.pages)
                self._offer(node)
            node = node.parent

    def insert(self, tokens, pages: List[int]) -> Tuple[List[int], RadixNode]:
        """Stores the whole pages of ``tokens``.  Returns (canonical page ids for those pages, deepest node):
        where the tree already held a page the caller must switch to the returned id and drop its own."""
        tokens = np.asarray(tokens, dtype=np.int32)
        n = len(tokens) // self.ps * self.ps
        tokens, pages = tokens[:n], list(pages[: n // self.ps])
        node, done = self._walk(tokens, split=True)
        canon = self._path_pages(node, done)
        if done < n:
            new_pages = pages[done // self.ps:]
            child = RadixNode(tokens[done:].copy(), list(new_pages), node)
            node.children[self._key(child.tokens)] = child
            self._nodes += 1
            self._evictable += len(new_pages)
            self._offer(child)
            self.pool.ref_pages(new_pages)
            self.metrics["inserted_pages"] += len(new_pages)
            # the previous tail of this path is no longer a tail
            self._retire_tail(node)
            self.pin_tail(child)
            canon = canon + new_pages
            node = child
        return canon, node

    def _tail_pages(self, node: RadixNode) -> List[int]:
        """Pages whose window storage a hit at the path's last aligned boundary (or at its end) would need."""
        n = node.path_len()
        pages = self._path_pages(node, n)
        boundary = n // self.align * self.align
        first = max(boundary - self.window, 0) // self.ps
        # a hit never resumes past the last aligned boundary, so the pages after it need no window storage
        return pages[first: boundary // self.ps]

    def _retire_tail(self, node: RadixNode) -> None:
        if node is self.root or not node.pages:
            return
        self.pool.unpin_swa(self._tail_pages(node), owner="tree")

    def pin_tail(self, node: RadixNode) -> None:
        """Keeps window storage alive for the tail of a cached path so that a later hit can resume there."""
        if node is self.root or not node.pages:
            return
        self.pool.pin_swa(self._tail_pages(node), owner="tree")

    def evictable_pages(self) -> int:
        """Pages held by unlocked nodes (kept incrementally)."""
        return self._evictable

    def _count_evictable(self) -> int:
        """The same figure from a full walk (tests compare the two)."""
        total, stack = 0, [self.root]
        while stack:
            nd = stack.pop()
            stack.extend(nd.children.values())
            if nd is not self.root and nd.lock_count == 0:
                total += len(nd.pages)
        return total

    def evict(self, n_pages: int) -> int:
        """Frees at least n_pages pages from unlocked leaves in LRU order (if available)."""
        freed = 0
        while self._lru and freed < n_pages:
            t, _, nd = heapq.heappop(self._lru)
            if nd.parent is None or nd.lock_count or not nd.is_leaf or t != nd.last_access:
                continue  # stale entry
            parent = nd.parent
            del parent.children[self._key(nd.tokens)]
            self.pool.unpin_swa(nd.pages, owner="tree")
            self.pool.unref_pages(nd.pages)
            freed += len(nd.pages)
            self._evictable -= len(nd.pages)
            self._nodes -= 1
            nd.parent = None
            if parent is not self.root:
                self._offer(parent)
        self.metrics["evicted_pages"] += freed
        return freed

    def reset(self) -> None:
        self.evict(1 << 60)

    def snapshot(self) -> dict:
        m = dict(self.metrics)
        m["hit_rate"] = m["hit_tokens"] / m["query_tokens"] if m["query_tokens"] else 0.0
        m["evictable_pages"] = self.evictable_pages()
        return m
