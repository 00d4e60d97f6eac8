"""Request, batch and context types shared by the scheduler, the engine and the model.

Counterpart of the reference's python/minisgl/core.py:21-253: ``SamplingParams`` (greedy iff
``(T<=0 or top_k==1) and top_p==1``), ``FlightLedger`` (launch / landing counters that hold a request's storage until
no forward that includes it is running), ``Req`` with its host token buffer, and ``Batch``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch

from .reasoning import ReasoningState, advance_reasoning_state, initial_reasoning_state


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    ignore_eos: bool = False
    max_tokens: int = 1024

    @property
    def is_greedy(self) -> bool:
        return (self.temperature <= 0.0 or self.top_k == 1) and self.top_p == 1.0


class FlightLedger:
    """Book-keeping of the forwards launched for one admitted request.

    With overlap scheduling a request can end (EOS, length, abort) while a forward that contains it is still running
    on the device; its pages, window slots and table row must stay untouched until that forward has landed.  The
    ledger counts launches and landings -- forwards of one rank land in launch order, so two counters are enough --
    and moves through three phases: ``open`` (may launch), ``closing`` (ended, waiting for landings) and ``closed``
    (storage returned).  The reference keeps a set of issue epochs for the same purpose
    (python/minisgl/core.py:33-97); ``admission`` plays the role of its generation id and guards against a landing
    that belongs to an earlier occupant of the same request object.
    """

    __slots__ = ("admission", "launched", "landed", "phase", "ended_because")

    def __init__(self, admission: int = -1):
        self.admission = admission
        self.launched = 0
        self.landed = 0
        self.phase = "open"
        self.ended_because: Optional[str] = None

    # -- forwards
    def launch(self) -> int:
        """Registers one forward; returns its ticket (to be handed back to :meth:`land`)."""
        if self.phase != "open":
            raise RuntimeError(f"request already ended ({self.ended_because}); no further forward may include it")
        self.launched += 1
        return self.launched - 1

    def land(self, admission: int, ticket: int) -> None:
        if admission != self.admission:
            raise RuntimeError(f"landing for admission {admission} reached a request of admission {self.admission}")
        if ticket != self.landed or ticket >= self.launched:
            raise RuntimeError(f"forward ticket {ticket} landed out of order (next expected {self.landed}, "
                               f"{self.launched} launched)")
        self.landed += 1

    @property
    def in_flight(self) -> int:
        return self.launched - self.landed

    # -- end of life
    @property
    def is_open(self) -> bool:
        return self.phase == "open"

    def end(self, because: str) -> None:
        if self.phase != "open":
            raise RuntimeError(f"request ended twice: first {self.ended_because!r}, now {because!r}")
        self.phase, self.ended_because = "closing", because

    @property
    def may_release(self) -> bool:
        """True exactly once: ended, nothing in flight, storage not yet returned."""
        return self.phase == "closing" and self.launched == self.landed

    def released(self) -> None:
        if not self.may_release:
            raise RuntimeError(f"storage release in phase {self.phase!r} with {self.in_flight} forward(s) in flight")
        self.phase = "closed"


@dataclass(eq=False)
class Req:
    """One admitted request.  ``input_ids`` is the host copy of prompt + committed output; ``cached_len`` counts the
    positions whose KV is in the cache, ``device_len`` the positions the device knows after the forward in
    preparation (cached + the rows that forward runs), ``max_device_len`` the prompt plus the output budget."""

    input_ids: torch.Tensor  # 1-D CPU int32
    table_idx: int
    cached_len: int
    output_len: int
    uid: int
    sampling_params: SamplingParams
    cache_handle: Any = None
    reasoning_effort: Optional[str] = None
    swa_evicted_seqlen: int = 0
    lifecycle: FlightLedger = field(default_factory=FlightLedger)
    pages: List[int] = field(default_factory=list)  # page ids in sequence order (owned or shared via the radix tree)

    def __post_init__(self) -> None:
        if self.input_ids.device.type != "cpu":
            raise ValueError("a request keeps its token ids on the host")
        n = len(self.input_ids)
        self.prompt_len = n
        self.device_len = n
        self.max_device_len = n + self.output_len
        if not (0 <= self.cached_len < n <= self.max_device_len):
            raise ValueError(f"inconsistent lengths: cached {self.cached_len}, prompt {n}, "
                             f"limit {self.max_device_len}")
        self._grow: Optional[torch.Tensor] = None   # preallocated host buffer, created at the first decode token
        self.reasoning_state = initial_reasoning_state(self.reasoning_effort)

    # -- lengths
    @property
    def extend_len(self) -> int:
        """Rows the next forward has to run to catch up with ``device_len``."""
        return self.device_len - self.cached_len

    @property
    def remain_len(self) -> int:
        return self.max_device_len - self.device_len

    @property
    def can_decode(self) -> bool:
        return self.device_len < self.max_device_len

    @property
    def can_commit_token(self) -> bool:
        return len(self.input_ids) < self.max_device_len

    def complete_one(self) -> None:
        """A forward covered everything up to ``device_len`` and sampled one more token."""
        self.cached_len, self.device_len = self.device_len, self.device_len + 1

    # -- host token buffer
    def append_host(self, next_token: torch.Tensor) -> None:
        """Appends one sampled token (a one-element CPU tensor of the ids' dtype) to the host copy."""
        if next_token.numel() != 1 or next_token.device.type != "cpu" or next_token.dtype != self.input_ids.dtype:
            raise ValueError("append_host expects one CPU token of the request's dtype")
        have = len(self.input_ids)
        if have >= self.max_device_len:
            raise RuntimeError("the request's output budget is used up")
        if self._grow is None:
            self._grow = torch.empty(self.max_device_len, dtype=self.input_ids.dtype)
            self._grow[:have] = self.input_ids
        self._grow[have] = next_token.view(())
        self.input_ids = self._grow[: have + 1]

    def observe_generated_token(self, token_id: int, *, think_end_token_id: int) -> None:
        self.reasoning_state = advance_reasoning_state(self.reasoning_state, token_id,
                                                       think_end_token_id=think_end_token_id)

    def __repr__(self) -> str:
        return (f"Req(uid={self.uid}, slot={self.table_idx}, cached={self.cached_len}, device={self.device_len}, "
                f"limit={self.max_device_len}, {self.lifecycle.phase})")


@dataclass
class Batch:
    reqs: List[Req]
    phase: str  # "prefill" | "decode"
    # filled by the scheduler / engine
    input_ids: Any = None        # [T] int32 device
    positions: Any = None        # [T] int32 device
    slots: Any = None            # [T] int32 device: request table slot of each row
    out_loc: Any = None          # [T] int32 device: token location of each row (page*page_size + offset)
    last_idx: Any = None         # [B] int64 device: row of each request's last token
    padded_reqs: List[Req] = field(default_factory=list)
    num_token_non_padded: int = 0
    reasoning_states: Any = None
    max_context: int = 0         # largest device_len in the batch (bounds index-surface widths)

    @property
    def is_prefill(self) -> bool:
        return self.phase == "prefill"

    @property
    def is_decode(self) -> bool:
        return self.phase == "decode"

    @property
    def size(self) -> int:
        return len(self.reqs)

    @property
    def padded_size(self) -> int:
        return len(self.padded_reqs) if self.padded_reqs else len(self.reqs)
