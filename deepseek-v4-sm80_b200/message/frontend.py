"""Messages consumed by the API frontend (python/minisgl/message/frontend.py:9-33)."""
from __future__ import annotations

from typing import Any, List, Optional

from .utils import message


@message
class UserReply:
    uid: int
    incremental_output: str
    finished: bool
    finish_reason: Optional[str] = None
    num_tokens: int = 0
    prompt_tokens: Optional[int] = None


@message
class BatchFrontendMsg:
    data: List[Any]
