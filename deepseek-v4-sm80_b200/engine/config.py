"""Engine configuration (python/minisgl/engine/config.py:16-72 of the reference).  Frozen; recipes and derived
values are written once by ``Engine._adjust_config`` through ``object.__setattr__``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch

from ..parallel.info import DistributedInfo
from ..utils.misc import UNSET


@dataclass(frozen=True)
class EngineConfig:
    model_path: str = ""
    tp_info: DistributedInfo = field(default_factory=lambda: DistributedInfo(0, 1))
    dtype: torch.dtype = torch.bfloat16
    max_running_req: Any = UNSET
    cuda_graph_bs: Optional[List[int]] = None
    cuda_graph_max_bs: Any = UNSET
    context_length: Any = UNSET
    recipe: Optional[str] = None
    page_size: int = 256
    memory_ratio: float = 0.9
    num_page_override: Optional[int] = None
    use_dummy_weight: bool = False
    use_pynccl: bool = True            # fused NVLink collectives (the reference's flag name); False = torch.distributed
    moe_mode: str = "ep"
    distributed_timeout: float = 60.0
    distributed_addr: Optional[str] = None
    device: str = "cuda"
    model_config: Any = None           # explicit ModelConfig (tests, benchmarks); else read from model_path
    enable_reasoning_sampler_contract: bool = False
    max_prefill_length: int = 8192
    seed: int = 0
    explicit_fields: frozenset = frozenset()

    @property
    def max_seq_len_override(self):
        return None if self.context_length is UNSET else self.context_length
