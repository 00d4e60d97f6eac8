"""Running (decoding) requests (python/minisgl/scheduler/decode.py:10-39)."""
from __future__ import annotations

from typing import List, Set

from ..core import Batch, Req


class DecodeManager:
    def __init__(self, page_size: int):
        self.page_size = page_size
        self.running: Set[Req] = set()

    def add(self, req: Req) -> None:
        if req.can_decode:
            self.running.add(req)

    def remove(self, req: Req) -> None:
        self.running.discard(req)

    def filter_reqs(self, reqs) -> None:
        """Keeps the requests of the last forward that can still decode."""
        for r in reqs:
            if r.can_decode and r.lifecycle.is_open:
                self.running.add(r)
            else:
                self.running.discard(r)

    @property
    def inflight_tokens(self) -> int:
        """Token capacity the running requests may still claim (each may also need a fresh page)."""
        return sum(r.remain_len + self.page_size - 1 for r in self.running)

    @property
    def runnable(self) -> bool:
        return bool(self.running)

    def schedule_next_batch(self) -> Batch | None:
        if not self.running:
            return None
        return Batch(sorted(self.running, key=lambda r: r.uid), "decode")
