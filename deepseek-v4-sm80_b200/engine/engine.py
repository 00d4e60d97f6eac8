"""The per-rank engine: owns the device, the communicator, the weights, the KV pools and the CUDA graphs, and runs
one forward per scheduled batch.

Start-up order (python/minisgl/engine/engine.py:147-284 of the reference, adapted): tensor-parallel info -> recipe /
config adjustment -> device and stream -> communication -> weights (checkpoint or random) -> graph-memory estimate ->
KV page count -> KV pools and page table -> sampler -> dummy request -> graph capture -> memory ledger check.
There is no BF16 weight-cache or Marlin repack stage: FP8 and FP4 weights are consumed in place.
"""
from __future__ import annotations

import dataclasses
import math
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ..core import Batch, Req
from ..dsv4_release import DSV4_RELEASE, RECIPES
from ..kvcache.pool import DSV4KVPool, PoolSizes, bytes_per_page, bytes_per_req_slot, bytes_per_swa_slot
from ..models.config import ModelConfig
from ..models.deepseek_v4 import DSV4Model, ForwardBatch, GreedyTail
from ..parallel import comm as comm_mod
from ..parallel.info import set_tp_info
from ..utils.logger import init_logger, set_log_rank
from ..utils.misc import UNSET, align_ceil, div_ceil
from . import graph_memory
from .config import EngineConfig
from .graph_policy import resolve_graph_buckets
from .sample import BatchSamplingArgs, ReasoningSampler, Sampler

logger = init_logger(__name__)


@dataclass
class ForwardOutput:
    next_tokens_gpu: torch.Tensor
    next_tokens_cpu: torch.Tensor
    copy_done_event: Any
    forward_ms: Optional[float] = None
    status: Any = None           # ops.native.StatusProbe whose snapshot was queued behind this forward (CUDA only)


def swa_slot_plan(max_running_req: int, prefill_budget: int, page_size: int, window: int) -> int:
    """Sliding-window slots to reserve: the pages of one full prefill forward, one spare, and per running request its
    hard share (:func:`minisgl.scheduler.cache.slots_per_request`: window pages, the page being written, the step
    overlap scheduling keeps in flight) plus ``ceil(window / ps)`` for the tail of the cached path it locks in the
    prefix tree.  Admission divides the pool by the hard share (``CacheManager.request_capacity``); the tree's part is
    an allowance that keeps prefix-hit resume points alive and is given up first under pressure.
    (The reference reserves at least 8 per request, python/minisgl/engine/engine.py:569-584.)"""
    from ..scheduler.cache import slots_per_request

    per_req = slots_per_request(window, page_size) + div_ceil(window, page_size)
    return div_ceil(prefill_budget, page_size) + 1 + max_running_req * per_req


class Engine:
    def __init__(self, config: EngineConfig):
        self.config = config = self._adjust_config(config)
        tp = config.tp_info
        set_tp_info(tp.rank, tp.size)
        set_log_rank(tp.rank)
        if config.device == "cuda":
            self.device = torch.device("cuda", self._local_device_index(tp.rank))
        else:
            self.device = torch.device(config.device)
        self.is_cuda = self.device.type == "cuda"
        if self.is_cuda:
            from ..utils.arch import require_blackwell

            require_blackwell(self.device.index)   # the kernels exist for sm_100a only: fail before touching weights
            torch.cuda.set_device(self.device)
            self.stream = torch.cuda.Stream(self.device)
        else:
            self.stream = None
        self.model_config: ModelConfig = config.model_config or self._load_model_config(config.model_path)
        cfg = self.model_config
        self.page_size = config.page_size
        self.cpu_group, self.comm = comm_mod.init_distributed(
            tp, self.device, config.distributed_addr, config.distributed_timeout, fused=config.use_pynccl,
            vocab_size=cfg.vocab_size, max_rows=max(config.max_prefill_length, config.max_running_req),
            hidden=cfg.hidden_size)
        free0 = self._sync_free_memory()
        t0 = time.time()
        self.weights = self._load_weights()
        self.weight_bytes = sum(v.numel() * v.element_size() for v in self.weights.values())
        logger.info_rank0("weights ready: %.2f GiB in %.1f s", self.weight_bytes / 2**30, time.time() - t0)
        self.graph_policy = resolve_graph_buckets(
            max_running_req=config.max_running_req, explicit_list=config.cuda_graph_bs,
            explicit_max=None if config.cuda_graph_max_bs is UNSET else config.cuda_graph_max_bs, enabled=self.is_cuda)
        self.context_classes = self._context_classes()
        self.graph_estimate = graph_memory.estimate_graph_memory(
            buckets=self.graph_policy.buckets, num_context_classes=len(self.context_classes),
            hidden_size=cfg.hidden_size)
        self.kv_plan = self._plan_kv()
        self.pool = DSV4KVPool(cfg, PoolSizes(self.kv_plan["num_pages"], self.kv_plan["swa_slots"],
                                              config.max_running_req, self.page_size), self.device)
        self.num_pages = self.kv_plan["num_pages"]
        self.max_seq_len = self.kv_plan["max_seq_len"]
        self.page_table = torch.zeros(config.max_running_req + 1, align_ceil(self.max_seq_len, self.page_size),
                                      dtype=torch.int32, device=self.device)
        self.dummy_slot = config.max_running_req
        ps = self.page_size
        row = self.pool.dummy_page * ps + torch.arange(self.page_table.shape[1], dtype=torch.int32) % ps
        self.page_table[self.dummy_slot] = row.to(self.device)
        self.last_token = torch.zeros(config.max_running_req + 1, dtype=torch.int32, device=self.device)
        self.model = DSV4Model(cfg, self.weights, self.pool, self.comm, config.moe_mode)
        self.model_prepare_report = self.model.prepare_report()
        logger.info_rank0("model prepared: %s", {k: v for k, v in self.model_prepare_report.items()
                                                 if k != "derived_bytes"})
        self.sampler: Sampler = Sampler(self.device, cfg.vocab_size, config.seed)
        self.reasoning_token_ids = None
        self.graph_runner = None
        self.status_probes = None
        self._probe_i = 0
        if self.is_cuda:
            from ..env import ENV
            from ..ops import native

            native.set_peer_wait_ms(ENV.PEER_WAIT_MS.value)
            if not ENV.DISABLE_STATUS_CHECK:
                self.status_probes = [native.StatusProbe(), native.StatusProbe()]
        self._events: List[Any] = []
        self.timings: List[Dict[str, Any]] = []
        self.record_timings = False
        if self.is_cuda and self.graph_policy.buckets:
            from .graph import GraphRunner

            before = torch.cuda.memory_allocated(self.device)
            self.graph_runner = GraphRunner(self)
            used = torch.cuda.memory_allocated(self.device) - before
            self.graph_memory_report = graph_memory.compare_graph_capture(self.graph_estimate, used)
        self.sync_all_ranks()

    # ------------------------------------------------------------------ configuration
    @staticmethod
    def _adjust_config(config: EngineConfig) -> EngineConfig:
        """Applies the recipe; values the user set explicitly win (python/minisgl/engine/engine.py:810-911)."""
        upd: Dict[str, Any] = {}
        recipe = config.recipe
        if recipe is not None:
            if recipe not in RECIPES:
                raise ValueError(f"unknown recipe {recipe!r}; choose from {sorted(RECIPES)}")
            mrr, gbs, ctx = RECIPES[recipe]
            if config.max_running_req is UNSET:
                upd["max_running_req"] = mrr
            if config.cuda_graph_max_bs is UNSET and not config.cuda_graph_bs:
                upd["cuda_graph_max_bs"] = min(gbs, upd.get("max_running_req", config.max_running_req
                                                            if config.max_running_req is not UNSET else mrr))
            if config.context_length is UNSET and ctx is not None:
                upd["context_length"] = ctx
        if config.max_running_req is UNSET and "max_running_req" not in upd:
            upd["max_running_req"] = RECIPES["default_m128"][0]
        if config.page_size <= 0 or config.page_size % 4:
            raise ValueError("page_size must be a positive multiple of 4")
        return dataclasses.replace(config, **upd) if upd else config

    @staticmethod
    def _local_device_index(rank: int) -> int:
        import os

        if "LOCAL_RANK" in os.environ:
            return int(os.environ["LOCAL_RANK"])
        return rank % max(torch.cuda.device_count(), 1)

    @staticmethod
    def _load_model_config(path: str) -> ModelConfig:
        from ..utils.hf import cached_load_hf_config

        return ModelConfig.from_hf(cached_load_hf_config(path))

    def _load_weights(self) -> Dict[str, torch.Tensor]:
        cfg, tp = self.model_config, self.config.tp_info
        if self.config.use_dummy_weight or not self.config.model_path:
            from ..models import synth

            from ..env import ENV

            return synth.random_weights(cfg, self.device, tp.rank, tp.size, self.config.moe_mode, self.config.seed,
                                        fast_experts=self.is_cuda,
                                        draw_on_host=self.is_cuda and bool(ENV.DUMMY_WEIGHT_ON_HOST))
        from ..models.weight import load_checkpoint
        from ..utils.hf import download_hf_weight

        return load_checkpoint(download_hf_weight(self.config.model_path), cfg, self.device, tp.rank, tp.size,
                               self.config.moe_mode)

    def _context_classes(self) -> List[int]:
        limit = self.config.max_seq_len_override or self.model_config.max_position
        classes = [c for c in (4 * self.model_config.index_topk, DSV4_RELEASE.graph_short_context) if c < limit]
        return classes + [limit]

    # ------------------------------------------------------------------ memory
    def _sync_free_memory(self) -> int:
        if not self.is_cuda:
            return 0
        torch.cuda.synchronize(self.device)
        free = torch.cuda.mem_get_info(self.device)[0]
        if self.cpu_group is not None:
            import torch.distributed as dist

            t = torch.tensor([free, -free], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.cpu_group)
            lo, hi = int(t[0]), -int(t[1])
            if hi - lo > 2 * 2**30:
                raise RuntimeError(f"free memory differs by {(hi - lo) / 2**30:.1f} GiB across ranks")
            free = lo
        return free

    def _plan_kv(self) -> Dict[str, int]:
        cfg, c = self.model_config, self.config
        ps = self.page_size
        limit = c.max_seq_len_override or cfg.max_position
        swa_slots = swa_slot_plan(c.max_running_req, c.max_prefill_length, ps, cfg.window_size)
        per_page = bytes_per_page(cfg, ps)
        fixed = swa_slots * bytes_per_swa_slot(cfg, ps) + (c.max_running_req + 1) * bytes_per_req_slot(cfg)
        want_pages = min(c.max_running_req * div_ceil(limit, ps) + div_ceil(c.max_prefill_length, ps), 1 << 18)
        if self.is_cuda:
            free = self._sync_free_memory()
            total = torch.cuda.get_device_properties(self.device).total_memory
            budget = free - int((1.0 - c.memory_ratio) * total) - fixed - self.graph_estimate.reserve_bytes
            table_bytes = (c.max_running_req + 1) * align_ceil(limit, ps) * 4
            budget -= table_bytes
            num_pages = graph_memory.select_num_pages(budget_bytes=budget, bytes_per_page=per_page,
                                                      override=c.num_page_override,
                                                      min_pages=div_ceil(c.max_prefill_length, ps) + 1)
            if c.num_page_override is None:
                num_pages = min(num_pages, want_pages)
        else:
            num_pages = c.num_page_override or min(want_pages, 256)
            swa_slots = min(swa_slots, num_pages)
        max_seq_len = min(limit, num_pages * ps)
        self.kv_capacity_plan_report = {
            "num_pages": num_pages, "kv_tokens": num_pages * ps, "swa_slots": swa_slots, "bytes_per_page": per_page,
            "fixed_bytes": fixed, "graph_reserve_bytes": self.graph_estimate.reserve_bytes,
            "weight_bytes": self.weight_bytes, "max_seq_len": max_seq_len,
        }
        logger.info_rank0("KV plan: %s", self.kv_capacity_plan_report)
        return {"num_pages": num_pages, "swa_slots": swa_slots, "max_seq_len": max_seq_len}

    # ------------------------------------------------------------------ sampler contract
    def enable_reasoning_sampler(self, token_ids) -> None:
        self.reasoning_token_ids = token_ids
        self.sampler = ReasoningSampler(self.device, self.model_config.vocab_size, token_ids, self.config.seed)

    # ------------------------------------------------------------------ forward
    def make_forward_batch(self, batch: Batch) -> ForwardBatch:
        return ForwardBatch(batch.input_ids, batch.positions, batch.slots, batch.out_loc, batch.last_idx,
                            self.page_table, batch.is_prefill, batch.max_context, None,
                            token_feedback=self.last_token if batch.is_decode else None)

    def forward_batch(self, batch: Batch, args: BatchSamplingArgs) -> ForwardOutput:
        t_ev = None
        if self.record_timings and self.is_cuda:
            t_ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            t_ev[0].record()
        # Greedy batches are sampled by the forward's last kernel (argmax over the vocabulary-parallel logits with
        # the shards' candidates exchanged in-kernel), which also stores the token as the request's next input.
        greedy = args.all_greedy and args.mask_ids is None
        toks = None
        if batch.is_decode and batch.input_ids is None:
            # decode rows take their token from last_token[slot] inside the embedding kernel, which fills this buffer
            batch.input_ids = torch.empty(batch.positions.shape[0], dtype=torch.int32, device=self.device)
        if self.graph_runner is not None and batch.is_decode and self.graph_runner.can_replay(batch):
            logits, toks = self.graph_runner.replay(batch)
            if not greedy:
                logits = self.comm.all_gather_last(logits)
        elif greedy:
            logits, toks = self.model.forward(self.make_forward_batch(batch), GreedyTail(self.last_token))
        else:
            logits = self.model.forward(self.make_forward_batch(batch))
        for req in batch.reqs:
            req.complete_one()
        if greedy:
            next_tokens = toks[: batch.size]
        else:
            next_tokens = self.sampler.sample(logits[: batch.size], args).to(torch.int32)
            # the sampled token is the next step's input: keep it on the device, per request slot
            sample_slots = batch.slots[: batch.size] if batch.is_decode else batch.slots[batch.last_idx]
            self.last_token[sample_slots.long()] = next_tokens
        probe = None
        if self.is_cuda:
            cpu = torch.empty(next_tokens.shape, dtype=next_tokens.dtype, pin_memory=True)
            cpu.copy_(next_tokens, non_blocking=True)
            if self.status_probes is not None:
                # two probes alternate: overlap scheduling keeps one forward in flight while the previous is read
                probe = self.status_probes[self._probe_i]
                self._probe_i ^= 1
                probe.snapshot()
            ev = torch.cuda.Event()
            ev.record()
        else:
            cpu, ev = next_tokens.clone(), None
        if t_ev is not None:
            t_ev[1].record()
            self.timings.append({"phase": batch.phase, "tokens": int(batch.num_token_non_padded),
                                 "reqs": batch.size, "events": t_ev})
        return ForwardOutput(next_tokens, cpu, ev, status=probe)

    # ------------------------------------------------------------------ misc
    def sync_all_ranks(self) -> None:
        if self.cpu_group is not None:
            import torch.distributed as dist

            dist.barrier(group=self.cpu_group)

    def shutdown(self) -> None:
        self.graph_runner = None
        import torch.distributed as dist

        if dist.is_initialized() and self.config.tp_info.size > 1:
            try:
                dist.destroy_process_group()
            except Exception:  # pragma: no cover
                pass
