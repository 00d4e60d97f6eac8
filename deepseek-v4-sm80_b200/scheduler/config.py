"""Scheduler configuration: the engine configuration plus the process-topology addresses
(python/minisgl/scheduler/config.py:15-43 of the reference)."""
from __future__ import annotations

import os
from dataclasses import dataclass

from ..engine.config import EngineConfig


def _unique(base: str) -> str:
    return f"ipc:///tmp/minisgl_b200_{base}.pid={os.getpid()}"


@dataclass(frozen=True)
class SchedulerConfig(EngineConfig):
    max_extend_tokens: int = 8192
    cache_type: str = "radix"
    offline_mode: bool = False
    stats_log_interval: float = 10.0
    disable_log_stats: bool = False
    heartbeat_name: str = ""          # shared-memory heartbeat board created by the server launcher ("" = none)
    heartbeat_timeout: float = 120.0  # seconds without a stamp, while busy, before a rank counts as wedged
    _unique_suffix: str = ""

    @property
    def zmq_backend_addr(self) -> str:      # tokenizer -> scheduler rank 0
        return f"ipc:///tmp/minisgl_b200_backend{self._unique_suffix}"

    @property
    def zmq_detokenizer_addr(self) -> str:  # scheduler rank 0 -> detokenizer
        return f"ipc:///tmp/minisgl_b200_detok{self._unique_suffix}"

    @property
    def zmq_scheduler_broadcast_addr(self) -> str:  # rank 0 -> other ranks
        return f"ipc:///tmp/minisgl_b200_bcast{self._unique_suffix}"
