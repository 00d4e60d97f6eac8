"""Generation-time wire protocol of DeepSeek-V4 chat: CHAT / THINKING / ANSWER.

A request that asked for reasoning starts in THINKING; the first ``</think>`` it generates moves it to
ANSWER.  The sampler uses the state to mask structural tokens (``<think>`` always, EOS while thinking,
``</think>`` otherwise).  Same contract as python/minisgl/reasoning.py:11-125 of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum


class ReasoningState(IntEnum):
    CHAT = 0
    THINKING = 1
    ANSWER = 2


@dataclass(frozen=True)
class ReasoningTokenIds:
    bos: int
    eos: int
    think_start: int
    think_end: int


def initial_reasoning_state(reasoning_effort) -> ReasoningState:
    if reasoning_effort is None or reasoning_effort == "none":
        return ReasoningState.CHAT
    if reasoning_effort in ("high", "max"):
        return ReasoningState.THINKING
    raise ValueError(f"reasoning_effort must be None, 'high', or 'max', got {reasoning_effort!r}")


def advance_reasoning_state(state: ReasoningState, token_id: int, *, think_end_token_id: int) -> ReasoningState:
    if state == ReasoningState.THINKING and token_id == think_end_token_id:
        return ReasoningState.ANSWER
    return state


def effective_reasoning_state(state: ReasoningState, *, current_input_token_id, think_end_token_id: int):
    """With overlap scheduling the host state lags the device by one token: if the token now entering the
    model is the closing delimiter, the sample that follows it is already an ANSWER sample."""
    if state == ReasoningState.THINKING and current_input_token_id == think_end_token_id:
        return ReasoningState.ANSWER
    return state


def _single_token_id(tokenizer, marker: str, label: str) -> int:
    enc = tokenizer.encode(marker, add_special_tokens=False)
    conv = tokenizer.convert_tokens_to_ids(marker)
    if not isinstance(enc, list) or len(enc) != 1:
        raise RuntimeError(f"reasoning sampler contract: {label} {marker!r} must encode to one token, got {enc!r}")
    if conv is None or int(conv) != int(enc[0]):
        raise RuntimeError(f"tokenizer lookup disagrees with encoding for {label} {marker!r}: {enc!r} vs {conv!r}")
    return int(enc[0])


def resolve_reasoning_token_ids(tokenizer) -> ReasoningTokenIds:
    if tokenizer.bos_token is None or tokenizer.bos_token_id is None:
        raise RuntimeError("tokenizer must define a BOS token and id")
    if tokenizer.eos_token is None or tokenizer.eos_token_id is None:
        raise RuntimeError("tokenizer must define an EOS token and id")
    bos = _single_token_id(tokenizer, tokenizer.bos_token, "BOS")
    eos = _single_token_id(tokenizer, tokenizer.eos_token, "EOS")
    if bos != int(tokenizer.bos_token_id) or eos != int(tokenizer.eos_token_id):
        raise RuntimeError("BOS/EOS encoding disagrees with the tokenizer's token ids")
    ids = ReasoningTokenIds(bos, eos, _single_token_id(tokenizer, "<think>", "opening marker"),
                            _single_token_id(tokenizer, "</think>", "closing marker"))
    vals = (ids.bos, ids.eos, ids.think_start, ids.think_end)
    if len(set(vals)) != 4:
        raise RuntimeError(f"reasoning structural token ids must be distinct, got {ids}")
    return ids
