"""Messages consumed by the scheduler (python/minisgl/message/backend.py:12-42)."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from ..core import SamplingParams
from .utils import message


@message
class UserMsg:
    uid: int
    input_ids: torch.Tensor        # 1-D int32 CPU
    sampling_params: SamplingParams
    reasoning_effort: Optional[str] = None


@message
class AbortBackendMsg:
    uid: int


@message
class ExitMsg:
    pass


@message
class BatchBackendMsg:
    data: List[Any]
