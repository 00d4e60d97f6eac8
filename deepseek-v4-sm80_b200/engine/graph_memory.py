"""Memory planning around CUDA-graph capture.

Before the KV pools are sized the engine needs an estimate of what graph capture will pin (activation workspaces
of the largest bucket plus per-graph bookkeeping); after capture the measured figure is compared with the plan and
an overrun aborts start-up instead of surfacing later as an allocation failure.  Same contract as the reference
(python/minisgl/engine/graph_memory.py:14-242); the constants are for this engine's kernels: activations per padded
row are ~0.6 MiB at hidden 4096 (residual streams, projections, 6 MoE route rows), graphs share one pool.
"""
from __future__ import annotations

from dataclasses import dataclass

MiB = 1 << 20

BASE_BYTES = 512 * MiB
PER_ROW_BYTES = 640 * 1024           # activation workspace per padded batch row (hidden 4096)
PER_GRAPH_BYTES = 24 * MiB
PER_EXTRA_CLASS_GRAPH_BYTES = 8 * MiB
MARGIN_BYTES = 512 * MiB


@dataclass(frozen=True)
class GraphMemoryEstimate:
    num_graphs: int
    max_bs: int
    estimate_bytes: int
    margin_bytes: int

    @property
    def reserve_bytes(self) -> int:
        return self.estimate_bytes + self.margin_bytes


def estimate_graph_memory(*, buckets, num_context_classes: int, hidden_size: int) -> GraphMemoryEstimate:
    if not buckets:
        return GraphMemoryEstimate(0, 0, 0, 0)
    max_bs = max(buckets)
    n = len(buckets) * num_context_classes
    act = PER_ROW_BYTES * max_bs * max(hidden_size, 256) // 4096
    est = BASE_BYTES + act + PER_GRAPH_BYTES * len(buckets) + PER_EXTRA_CLASS_GRAPH_BYTES * len(buckets) * (
        num_context_classes - 1)
    return GraphMemoryEstimate(n, max_bs, int(est), MARGIN_BYTES)


def select_num_pages(*, budget_bytes: int, bytes_per_page: int, override=None, min_pages: int = 2) -> int:
    """Pages that fit the budget.  An explicit override is honoured or rejected, never silently changed."""
    fit = max(int(budget_bytes // max(bytes_per_page, 1)), 0)
    if override is not None:
        if override < min_pages:
            raise ValueError(f"num_pages override {override} is below the minimum {min_pages}")
        if override > fit:
            raise RuntimeError(f"num_pages override {override} does not fit: only {fit} pages fit in "
                               f"{budget_bytes / MiB:.0f} MiB")
        return int(override)
    if fit < min_pages:
        raise RuntimeError(f"not enough memory for the KV cache: {fit} pages fit, {min_pages} needed")
    return fit


def compare_graph_capture(estimate: GraphMemoryEstimate, actual_bytes: int) -> dict:
    report = {"estimate_bytes": estimate.estimate_bytes, "margin_bytes": estimate.margin_bytes,
              "actual_bytes": int(actual_bytes), "overrun_bytes": max(int(actual_bytes) - estimate.reserve_bytes, 0)}
    if report["overrun_bytes"] > 0:
        raise RuntimeError("CUDA graph capture used %.1f MiB, more than the planned %.1f MiB (+%.1f MiB margin)" % (
            actual_bytes / MiB, estimate.estimate_bytes / MiB, estimate.margin_bytes / MiB))
    return report
