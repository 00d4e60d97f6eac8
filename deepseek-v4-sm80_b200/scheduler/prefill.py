"""Resident chunked prefill.

Every admitted prompt stays *resident* until its last chunk ran; each prefill forward spends one token budget
(8 192 by default) across all resident prompts with bounded max-min fairness in page-size quanta, so a very long
prompt cannot starve short ones and every resident prompt progresses in every forward
(python/minisgl/scheduler/prefill.py:32-115 and :275-411 of the reference).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, List, Optional, Sequence

import torch

from ..core import Batch, Req, SamplingParams
from ..utils.misc import div_ceil
from .cache import CacheManager
from .table import TableManager


def allocate_fair_prefill_chunks(*, token_budget: int, alignment_quantum: int, scheduled_tokens: Sequence[int],
                                 remaining_tokens: Sequence[int]) -> List[int]:
    """Splits one forward's token budget.  Every request first gets one quantum (or its final tail); then, in rounds,
    every unfinished request gets another quantum, visited in order of least granted progress (FIFO index breaks
    ties), until the budget is spent.  A grant smaller than a quantum is only ever a request's final tail -- except
    when the whole budget is below one quantum."""
    if token_budget <= 0 or alignment_quantum <= 0:
        raise ValueError("token_budget and alignment_quantum must be positive")
    if len(scheduled_tokens) != len(remaining_tokens):
        raise ValueError("scheduled_tokens and remaining_tokens must have equal length")
    if any(v < 0 for v in scheduled_tokens) or any(v <= 0 for v in remaining_tokens):
        raise ValueError("scheduled_tokens must be >= 0 and remaining_tokens > 0")
    n = len(remaining_tokens)
    grant = [0] * n
    left = int(token_budget)
    q = alignment_quantum
    for i in range(n):  # first share
        if left <= 0:
            break
        g = min(remaining_tokens[i], q if left >= q else left)
        grant[i], left = g, left - g
    while left > 0:
        order = sorted((i for i in range(n) if 0 < grant[i] < remaining_tokens[i]),
                       key=lambda i: (scheduled_tokens[i] + grant[i], i))
        progressed = False
        for i in order:
            rest = remaining_tokens[i] - grant[i]
            step = rest if rest < q else q
            if step > left:
                continue
            grant[i] += step
            left -= step
            progressed = True
            if left <= 0:
                break
        if not progressed:
            break
    assert sum(grant) <= token_budget
    return grant


@dataclass
class PendingReq:
    uid: int
    input_ids: torch.Tensor
    sampling_params: SamplingParams
    reasoning_effort: Optional[str] = None

    @property
    def input_len(self) -> int:
        return len(self.input_ids)

    @property
    def output_len(self) -> int:
        return self.sampling_params.max_tokens


class PrefillManager:
    def __init__(self, cache: CacheManager, table: TableManager, decode, page_size: int, max_seq_len: int):
        self.cache, self.table, self.decode = cache, table, decode
        self.ps, self.max_seq_len = page_size, max_seq_len
        self.slot_budget = 0                   # prefill token budget the window-slot plan assumes (set per schedule)
        self.pending: Deque[PendingReq] = deque()
        self.resident: List[Req] = []          # admitted, prefill not finished (FIFO)
        self.generation = 0
        self.deferred_chunks = 0
        self.shrunk_chunks = 0

    def add_one_req(self, p: PendingReq) -> None:
        self.pending.append(p)

    @property
    def runnable(self) -> bool:
        return bool(self.pending) or bool(self.resident)

    def abort(self, uid: int) -> Optional[Req]:
        for p in list(self.pending):
            if p.uid == uid:
                self.pending.remove(p)
                return None
        for r in self.resident:
            if r.uid == uid:
                self.resident.remove(r)
                return r
        return None

    # ------------------------------------------------------------------ admission
    def _claimed_pages(self) -> int:
        active = list(self.resident) + list(self.decode.running)
        return sum(self.cache.pages_still_needed(r) for r in active)

    def _try_admit(self, p: PendingReq) -> Optional[Req]:
        if self.table.available_size == 0:
            return None
        m = self.cache.match_req(p.input_ids)
        total_pages = div_ceil(p.input_len + p.output_len, self.ps)
        need = total_pages - m.length // self.ps
        # the matched pages may be counted as evictable right now; once adopted they are locked, so they cannot pay
        # for anybody's future pages
        if need + self._claimed_pages() > self.cache.available_pages - len(m.pages):
            return None
        # window slots are a second, much smaller resource: every admitted request keeps a bounded number pinned
        active = len(self.resident) + len(self.decode.running)
        if active + 1 > self.cache.request_capacity(self.slot_budget):
            return None
        slot = self.table.allocate()
        req = Req(input_ids=p.input_ids, table_idx=slot, cached_len=m.length, output_len=p.output_len, uid=p.uid,
                  sampling_params=p.sampling_params, reasoning_effort=p.reasoning_effort)
        self.generation += 1
        req.lifecycle.admission = self.generation
        req.prefill_granted = 0
        self.cache.adopt_prefix(req, m)
        return req

    # ------------------------------------------------------------------ scheduling
    def schedule_next_batch(self, budget: int) -> Optional[Batch]:
        self.slot_budget = budget
        # admit while the budget can still give every resident prompt a share
        while self.pending and len(self.resident) * min(self.ps, budget) < budget:
            req = self._try_admit(self.pending[0])
            if req is None:
                break
            self.pending.popleft()
            self.resident.append(req)
        if not self.resident:
            return None
        max_reqs = max(budget // min(self.ps, budget), 1)
        chosen = self.resident[:max_reqs]
        grants = allocate_fair_prefill_chunks(
            token_budget=budget, alignment_quantum=min(self.ps, budget),
            scheduled_tokens=[r.prefill_granted for r in chosen], remaining_tokens=[r.extend_len for r in chosen])
        reqs, chunks = [], []
        for r, g in zip(chosen, grants):
            if g <= 0:
                continue
            q = min(self.ps, budget)
            while g > 0 and not self.cache.try_allocate(r, r.cached_len + g):
                # no storage for the whole share right now (other requests still pin it): take a smaller piece,
                # whole quanta only, or wait for a later forward
                g = (g // 2) // q * q
                self.shrunk_chunks += 1
            if g <= 0:
                self.deferred_chunks += 1
                continue
            r.prefill_granted += g
            reqs.append(r)
            chunks.append(g)
        if not reqs:
            return None
        batch = Batch(reqs, "prefill")
        batch.chunk_lens = chunks
        batch.is_final = [r.cached_len + g == r.device_len for r, g in zip(reqs, chunks)]
        # rotate: unfinished prompts that ran go behind the ones that did not get a share
        finished = {id(r) for r, f in zip(reqs, batch.is_final) if f}
        ran = {id(r) for r in reqs}
        self.resident = [r for r in self.resident if id(r) not in ran] + \
                        [r for r in self.resident if id(r) in ran and id(r) not in finished]
        return batch
