"""Request, batch and context types shared by the scheduler, the engine and the model.

Counterpart of the reference's python/minisgl/core.py:21-253: ``SamplingParams`` (greedy iff
``(T<=0 or top_k==1) and top_p==1``), the per-request lifecycle ledger that defers resource release until
every issued forward has completed, ``Req`` with its host token buffer, and ``Batch``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, auto
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


class RequestLifecycleState(Enum):
    ACTIVE = auto()
    TERMINAL_PENDING_RETIRE = auto()
    RETIRED = auto()


@dataclass
class RequestLifecycle:
    """Which forwards were issued for a request generation and whether its terminal status is committed."""

    generation_id: int = -1
    state: RequestLifecycleState = RequestLifecycleState.ACTIVE
    next_issue_epoch: int = 0
    outstanding_epochs: set = field(default_factory=set)
    terminal_finish_reason: Optional[str] = None
    resources_released: bool = False

    def issue(self) -> int:
        if self.state is not RequestLifecycleState.ACTIVE:
            raise RuntimeError(f"cannot issue forward for request in lifecycle state {self.state.name}")
        e = self.next_issue_epoch
        self.next_issue_epoch += 1
        self.outstanding_epochs.add(e)
        return e

    def complete(self, *, generation_id: int, issue_epoch: int) -> None:
        if generation_id != self.generation_id:
            raise RuntimeError(f"request generation mismatch: expected={self.generation_id}, got={generation_id}")
        if issue_epoch not in self.outstanding_epochs:
            raise RuntimeError(f"request issue epoch {issue_epoch} is not outstanding")
        self.outstanding_epochs.remove(issue_epoch)

    def commit_terminal(self, finish_reason: str) -> None:
        if self.state is not RequestLifecycleState.ACTIVE:
            raise RuntimeError(f"terminal status may be committed exactly once; state is {self.state.name}")
        self.state = RequestLifecycleState.TERMINAL_PENDING_RETIRE
        self.terminal_finish_reason = finish_reason

    @property
    def accepts_completion(self) -> bool:
        return self.state is RequestLifecycleState.ACTIVE

    @property
    def ready_to_release_resources(self) -> bool:
        return (self.state is RequestLifecycleState.TERMINAL_PENDING_RETIRE and not self.outstanding_epochs
                and not self.resources_released)

    def mark_resources_released(self) -> None:
        if not self.ready_to_release_resources:
            raise RuntimeError("request resources may retire only once after all issued forwards complete")
        self.resources_released = True
        self.state = RequestLifecycleState.RETIRED


@dataclass(eq=False)
class Req:
    input_ids: torch.Tensor  # 1-D CPU int32 tensor: prompt + committed output tokens
    table_idx: int
    cached_len: int
    output_len: int
    uid: int
    sampling_params: SamplingParams
    cache_handle: Any = None
    reasoning_effort: Optional[str] = None
    swa_evicted_seqlen: int = 0
    lifecycle: RequestLifecycle = field(default_factory=RequestLifecycle)
    pages: List[int] = field(default_factory=list)  # page ids in sequence order (owned or shared via the radix tree)

    def __post_init__(self) -> None:
        assert self.input_ids.device.type == "cpu"
        self.device_len = len(self.input_ids)
        self.max_device_len = len(self.input_ids) + self.output_len
        assert 0 <= self.cached_len < self.device_len <= self.max_device_len
        self.prompt_len = len(self.input_ids)
        self.reasoning_state = initial_reasoning_state(self.reasoning_effort)
        self._host_buf: Optional[torch.Tensor] = None

    def observe_generated_token(self, token_id: int, *, think_end_token_id: int) -> None:
        self.reasoning_state = advance_reasoning_state(self.reasoning_state, token_id,
                                                       think_end_token_id=think_end_token_id)

    @property
    def remain_len(self) -> int:
        return self.max_device_len - self.device_len

    @property
    def extend_len(self) -> int:
        return self.device_len - self.cached_len

    def complete_one(self) -> None:
        self.cached_len = self.device_len
        self.device_len += 1

    def append_host(self, next_token: torch.Tensor) -> None:
        """Commits one sampled token to the host copy; the buffer is allocated once, on the first decode."""
        if next_token.device.type != "cpu" or next_token.dtype != self.input_ids.dtype or next_token.numel() != 1:
            raise ValueError("append_host expects one CPU token of the request's dtype")
        n = len(self.input_ids)
        if n >= self.max_device_len:
            raise RuntimeError("request has no remaining host token capacity")
        if self._host_buf is None:
            self._host_buf = torch.empty(self.max_device_len, dtype=self.input_ids.dtype)
            self._host_buf[:n].copy_(self.input_ids)
        self._host_buf[n] = next_token.reshape(())
        self.input_ids = self._host_buf[: n + 1]

    @property
    def can_decode(self) -> bool:
        return self.remain_len > 0

    @property
    def can_commit_token(self) -> bool:
        return len(self.input_ids) < self.max_device_len

    def __repr__(self) -> str:
        return (f"Req(uid={self.uid}, table_idx={self.table_idx}, cached_len={self.cached_len}, "
                f"device_len={self.device_len}, max_device_len={self.max_device_len})")


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
