"""Arbitration between prefill and decode forwards under mixed load.

Contract (python/minisgl/scheduler/phase_policy.py:8-110 of the reference): with only one phase runnable it runs
(an isolated prefill gets the full budget).  When both are runnable: the first conflict goes to decode; two prefills
never run back to back; after ``max_consecutive_decode`` decodes one prefill runs with the smaller mixed budget.
The state only advances when the scheduler reports that the chosen batch was really built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

MIXED_PREFILL_BUDGET = 2048
MAX_CONSECUTIVE_DECODE = 4


@dataclass(frozen=True)
class PhaseDecision:
    phase: Optional[str]
    prefill_budget: int = 0
    mixed: bool = False


class MixedPhaseFairPolicy:
    def __init__(self, *, isolated_prefill_budget: int, mixed_prefill_budget: int = MIXED_PREFILL_BUDGET,
                 max_consecutive_decode: int = MAX_CONSECUTIVE_DECODE, first_conflict: str = "decode"):
        if isolated_prefill_budget <= 0 or mixed_prefill_budget <= 0 or max_consecutive_decode <= 0:
            raise ValueError("budgets and max_consecutive_decode must be positive")
        if first_conflict not in ("prefill", "decode"):
            raise ValueError("first_conflict must be 'prefill' or 'decode'")
        self.isolated_prefill_budget = int(isolated_prefill_budget)
        self.mixed_prefill_budget = min(int(mixed_prefill_budget), self.isolated_prefill_budget)
        self.max_consecutive_decode = int(max_consecutive_decode)
        self.first_conflict = first_conflict
        self.reset_mixed_state()

    def reset_mixed_state(self) -> None:
        self._active, self._last, self._decodes = False, None, 0

    def choose(self, *, prefill_runnable: bool, decode_runnable: bool) -> PhaseDecision:
        if not (prefill_runnable or decode_runnable):
            return PhaseDecision(None)
        if not decode_runnable:
            return PhaseDecision("prefill", self.isolated_prefill_budget)
        if not prefill_runnable:
            return PhaseDecision("decode")
        if not self._active:
            phase = self.first_conflict
        elif self._last == "prefill" or self._decodes < self.max_consecutive_decode:
            phase = "decode"
        else:
            phase = "prefill"
        return PhaseDecision(phase, self.mixed_prefill_budget if phase == "prefill" else 0, mixed=True)

    def record_scheduled(self, phase: Optional[str], *, prefill_runnable: bool, decode_runnable: bool) -> None:
        if phase is None or not (prefill_runnable and decode_runnable):
            self.reset_mixed_state()
            return
        self._active, self._last = True, phase
        self._decodes = self._decodes + 1 if phase == "decode" else 0

    def snapshot(self) -> dict:
        return {"mixed_active": self._active, "last_mixed_phase": self._last,
                "consecutive_mixed_decode": self._decodes, "isolated_prefill_budget": self.isolated_prefill_budget,
                "mixed_prefill_budget": self.mixed_prefill_budget,
                "max_consecutive_decode": self.max_consecutive_decode, "first_conflict": self.first_conflict}
