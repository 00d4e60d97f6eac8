"""Tensor-parallel rank bookkeeping (python/minisgl/distributed/info.py of the reference)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class DistributedInfo:
    rank: int
    size: int

    def __post_init__(self):
        assert 0 <= self.rank < self.size

    def is_primary(self) -> bool:
        return self.rank == 0


_TP_INFO: Optional[DistributedInfo] = None


def set_tp_info(rank: int, size: int) -> None:
    global _TP_INFO
    _TP_INFO = DistributedInfo(rank, size)


def get_tp_info() -> DistributedInfo:
    return _TP_INFO if _TP_INFO is not None else DistributedInfo(0, 1)


def try_get_tp_info() -> Optional[DistributedInfo]:
    return _TP_INFO
