"""Frozen release policy: the values every recipe shares (python/minisgl/dsv4_release.py:25-33 of the reference,
re-derived for B200: there is no Marlin repack step to time and no BF16 weight cache to build)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class DSV4ReleasePolicy:
    page_size: int = 256
    prefill_budget: int = 8192
    mixed_prefill_budget: int = 2048
    max_consecutive_decode: int = 4
    comm_buffer_bytes: int = 32 << 20       # symmetric buffer: messages up to this size use the fused P2P kernels
    graph_short_context: int = 32768        # first CUDA-graph context class; the second is the model limit
    moe_mode: str = "ep"                    # experts sharded by id across ranks (tp = by intermediate column)
    page_clear_scope: str = "component"


DSV4_RELEASE = DSV4ReleasePolicy()

RECIPES = {
    # name: (max_running_req, cuda_graph_max_bs, context_length)
    "default_m128": (128, 128, None),
    "low_m64": (64, 64, None),
    "high_m256": (256, 256, None),
    "long_context_m8": (8, 8, 1048576),
}
