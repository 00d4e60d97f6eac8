"""Request-slot free list (python/minisgl/scheduler/table.py:4-21).  The page table itself lives in the engine."""
from __future__ import annotations

from typing import List


class TableManager:
    def __init__(self, max_running_req: int):
        self.max_running_req = max_running_req
        self._free: List[int] = list(range(max_running_req - 1, -1, -1))

    @property
    def available_size(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise RuntimeError("no free request slot")
        return self._free.pop()

    def free(self, slot: int) -> None:
        assert 0 <= slot < self.max_running_req and slot not in self._free, f"bad slot free: {slot}"
        self._free.append(slot)
