"""CUDA-graph decode replay.

One set of static input buffers sized for the largest bucket; one captured graph per (batch-size bucket, context
class).  A context class fixes the host-side constants a decode forward depends on -- whether the indexer needs
logits at all (contexts up to 4 x top-k keep every compressed entry) and how wide its logits workspace is -- so short
contexts do not pay for million-token metadata.  Everything else a step needs (page table, SWA map, last sampled
tokens) lives in fixed device buffers that the kernels read directly, so there is no per-replay metadata pass.
Counterpart of python/minisgl/engine/graph.py:37-677 of the reference (32 K + model-width classes, buckets padded
with a dummy request); a third, small class covers contexts where top-k selection is the identity.
"""
from __future__ import annotations

import bisect
from typing import Dict, List, Optional, Tuple

import torch

from ..core import Batch
from ..models.deepseek_v4 import ForwardBatch, GreedyTail
from ..ops import native
from ..utils.logger import init_logger
from .graph_policy import pick_bucket

logger = init_logger(__name__)


class GraphCaptureBuffer:
    """Static inputs and outputs of the captured decode graphs.  The per-step inputs sit in one int32 block
    [4, max_bs] (positions, request slots, token locations, and the number of valid rows in [3, 0]) that one copy
    fills from the block the scheduler uploaded.  Token ids are not an input: the graph's embedding kernel gathers
    them from the engine's device-resident feedback buffer and leaves them in ``input_ids``; the graph's last
    kernel writes the greedy tokens to ``next_tokens``."""

    def __init__(self, max_bs: int, device):
        z = dict(dtype=torch.int32, device=device)
        self.block = torch.zeros(4, max_bs, **z)
        self.positions, self.slots, self.out_loc = self.block[0], self.block[1], self.block[2]
        self.num_valid = self.block[3, :1]
        self.input_ids = torch.zeros(max_bs, **z)
        self.next_tokens = torch.zeros(max_bs, **z)
        self.logits = None    # [max_bs, vocab / tp] fp32, shared by all graphs (set by the runner)

    def copy_from(self, batch: Batch, bs: int) -> None:
        blk = getattr(batch, "device_block", None)
        if blk is not None and blk.shape == (4, bs):
            self.block[:, :bs].copy_(blk, non_blocking=True)      # one strided copy for everything
            return
        self.positions[:bs].copy_(batch.positions[:bs], non_blocking=True)
        self.slots[:bs].copy_(batch.slots[:bs], non_blocking=True)
        self.out_loc[:bs].copy_(batch.out_loc[:bs], non_blocking=True)
        self.num_valid.fill_(batch.num_token_non_padded)


class GraphRunner:
    def __init__(self, engine):
        self.engine = engine
        self.buckets: List[int] = list(engine.graph_policy.buckets)
        self.classes: List[int] = list(engine.context_classes)
        self.max_bs = max(self.buckets)
        self.buffer = GraphCaptureBuffer(self.max_bs, engine.device)
        # every graph writes its logits shard into the same static buffer: a per-graph output would pin
        # bucket x vocab floats for each of the dozens of (bucket, context class) graphs of a serving recipe
        self.buffer.logits = torch.empty(self.max_bs, engine.weights["head.weight"].shape[0], dtype=torch.float32,
                                         device=engine.device)
        self.graphs: Dict[Tuple[int, int], torch.cuda.CUDAGraph] = {}
        self.logits: Dict[Tuple[int, int], torch.Tensor] = {}
        self.launches: Dict[Tuple[int, int], int] = {}
        self.pool = None
        self.capture_status = {"captured": 0, "replays": 0, "eager_decode": 0, "unsupported_bs": 0,
                               "context_overflow": 0, "buckets": self.buckets, "classes": self.classes}
        self._capture_all()

    # ------------------------------------------------------------------ capture
    def _forward(self, bs: int, max_context: int):
        """One decode forward on the static buffers: (this rank's logits shard [bs, vocab / tp], greedy tokens)."""
        b, e = self.buffer, self.engine
        fb = ForwardBatch(b.input_ids[:bs], b.positions[:bs], b.slots[:bs], b.out_loc[:bs], None, e.page_table,
                          False, max_context, b.num_valid, token_feedback=e.last_token)
        return e.model.forward(fb, GreedyTail(e.last_token, b.next_tokens[:bs], b.logits[:bs]))

    def _capture_all(self) -> None:
        e = self.engine
        b = self.buffer
        b.slots.fill_(e.dummy_slot)
        b.out_loc.fill_(e.pool.dummy_page * e.page_size)
        b.num_valid.fill_(1)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        for bs in sorted(self.buckets, reverse=True):
            for ci, limit in enumerate(self.classes):
                with torch.cuda.stream(stream):
                    self._forward(bs, limit)  # warm-up: lazy attribute setup, cached conversions
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                n0 = native.launch_count()
                with torch.cuda.graph(g, pool=self.pool, stream=stream):
                    out = self._forward(bs, limit)
                self.launches[(bs, ci)] = native.launch_count() - n0
                if self.pool is None:
                    self.pool = g.pool()
                self.graphs[(bs, ci)] = g
                self.logits[(bs, ci)] = out[0]
                self.capture_status["captured"] += 1
        torch.cuda.synchronize()
        native.assert_device_ok()
        logger.info_rank0("captured %d CUDA graphs (buckets %s, context classes %s)", len(self.graphs), self.buckets,
                          self.classes)

    # ------------------------------------------------------------------ replay
    def padded_size(self, bs: int) -> int:
        b = pick_bucket(self.buckets, bs)
        return b if b is not None else bs

    def _class_of(self, max_context: int) -> Optional[int]:
        i = bisect.bisect_left(self.classes, max_context)
        return i if i < len(self.classes) else None

    def can_replay(self, batch: Batch) -> bool:
        if not batch.is_decode:
            return False
        if pick_bucket(self.buckets, batch.size) is None:
            self.capture_status["unsupported_bs"] += 1
            return False
        if self._class_of(batch.max_context) is None:
            self.capture_status["context_overflow"] += 1
            return False
        return True

    def replay(self, batch: Batch):
        """Returns (this rank's logits shard of the padded batch, greedy tokens int32 [bucket]); the graph has
        already stored the greedy tokens as next-step feedback."""
        bs = pick_bucket(self.buckets, batch.size)
        ci = self._class_of(batch.max_context)
        if bs is None or ci is None:
            raise RuntimeError("decode batch has no captured graph; call can_replay first")
        assert batch.positions.shape[0] == bs, "decode batch must be padded to its bucket"
        self.buffer.copy_from(batch, bs)
        self.graphs[(bs, ci)].replay()
        native.add_launches(self.launches[(bs, ci)])
        self.capture_status["replays"] += 1
        return self.logits[(bs, ci)], self.buffer.next_tokens[:bs]
