"""Messages consumed by the tokenizer / detokenizer workers (python/minisgl/message/tokenizer.py:11-48)."""
from __future__ import annotations

from typing import Any, List, Optional

from ..core import SamplingParams
from .utils import message

message(SamplingParams)


@message
class TokenizeMsg:
    uid: int
    text: Any                      # str prompt or list of chat messages
    sampling_params: SamplingParams
    reasoning_effort: Optional[str] = None


@message
class AbortMsg:
    uid: int


@message
class DetokenizeMsg:
    uid: int
    next_token: int
    finished: bool
    finish_reason: Optional[str] = None
    prompt_tokens: Optional[int] = None   # set on a request's first reply (for the usage record)


@message
class BatchTokenizerMsg:
    data: List[Any]
