"""Which decode batch sizes get a CUDA graph.

Pure function of the configuration, as in the reference (python/minisgl/engine/graph_policy.py:37-176): the release
default is ``1, 2, 4, 8..256 step 8, 272.. step 16`` up to the endpoint (at most 512); an explicit list or an explicit
maximum may replace it; every bucket must be <= max_running_req.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

MAX_GRAPH_BS = 512


@dataclass(frozen=True)
class GraphBucketPolicy:
    mode: str                 # explicit_list | explicit_max | release_default | disabled
    buckets: tuple
    max_bs: int


def default_buckets(endpoint: int) -> List[int]:
    if endpoint <= 0:
        return []
    out = [b for b in (1, 2, 4) if b <= endpoint]
    out += list(range(8, min(endpoint, 256) + 1, 8))
    out += list(range(272, endpoint + 1, 16))
    if out and out[-1] != endpoint:
        out.append(endpoint)
    if not out:
        out = [endpoint]
    return sorted(set(out))


def resolve_graph_buckets(*, max_running_req: int, explicit_list: Optional[Sequence[int]] = None,
                          explicit_max: Optional[int] = None, enabled: bool = True) -> GraphBucketPolicy:
    if not enabled or explicit_max == 0:
        return GraphBucketPolicy("disabled", (), 0)
    if explicit_list:
        b = sorted(set(int(x) for x in explicit_list))
        if b[0] <= 0:
            raise ValueError("cuda graph batch sizes must be positive")
        if b[-1] > max_running_req:
            raise ValueError(f"cuda graph batch size {b[-1]} exceeds max_running_req {max_running_req}")
        if b[-1] > MAX_GRAPH_BS:
            raise ValueError(f"cuda graph batch size {b[-1]} exceeds the supported maximum {MAX_GRAPH_BS}")
        return GraphBucketPolicy("explicit_list", tuple(b), b[-1])
    if explicit_max is not None:
        if explicit_max < 0:
            raise ValueError("cuda_graph_max_bs must be >= 0")
        if explicit_max > max_running_req:
            raise ValueError(f"cuda_graph_max_bs {explicit_max} exceeds max_running_req {max_running_req}")
        if explicit_max > MAX_GRAPH_BS:
            raise ValueError(f"cuda_graph_max_bs {explicit_max} exceeds the supported maximum {MAX_GRAPH_BS}")
        return GraphBucketPolicy("explicit_max", tuple(default_buckets(explicit_max)), explicit_max)
    endpoint = min(max_running_req, MAX_GRAPH_BS)
    return GraphBucketPolicy("release_default", tuple(default_buckets(endpoint)), endpoint)


def pick_bucket(buckets: Sequence[int], bs: int) -> Optional[int]:
    for b in buckets:
        if b >= bs:
            return b
    return None
