"""Interval throughput counters for the periodic scheduler log line (python/minisgl/scheduler/stats.py:7-57)."""
from __future__ import annotations

import time


class StatsTracker:
    def __init__(self, interval: float = 10.0, clock=time.monotonic):
        self.interval, self.clock = interval, clock
        self.t0 = clock()
        self.prompt_tokens = self.gen_tokens = 0
        self.total_prompt = self.total_gen = 0
        self.prefill_steps = self.decode_steps = 0

    def on_prefill(self, n: int) -> None:
        self.prompt_tokens += n
        self.total_prompt += n
        self.prefill_steps += 1

    def on_decode(self, n: int) -> None:
        self.gen_tokens += n
        self.total_gen += n
        self.decode_steps += 1

    def maybe_report(self, running: int, waiting: int, kv_used: float):
        now = self.clock()
        dt = now - self.t0
        if dt < self.interval:
            return None
        line = (f"prompt {self.prompt_tokens / dt:.1f} tok/s | generation {self.gen_tokens / dt:.1f} tok/s | "
                f"running {running} | waiting {waiting} | KV {kv_used * 100:.1f}%")
        self.t0, self.prompt_tokens, self.gen_tokens = now, 0, 0
        return line
