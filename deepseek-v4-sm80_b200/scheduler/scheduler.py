"""Per-rank scheduler: admits requests, arbitrates prefill vs decode, prepares device inputs, launches the forward and
commits results, with *overlap scheduling* -- batch N+1 is scheduled and launched while batch N's sampled tokens are
still on their way to the host.  Counterpart of python/minisgl/scheduler/scheduler.py:62-573 of the reference.

Every rank runs this loop on identical messages (rank 0 re-publishes what it receives), so all ranks build identical
batches without any device-side coordination.  Host->device traffic per step is one pinned int32 block
(positions, slots, token locations, and for prefill the chunk's token ids); device->host is the sampled tokens.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..core import Batch, Req
from ..engine.engine import Engine, ForwardOutput
from ..engine.sample import BatchSamplingArgs, ReasoningSampler
from ..message import AbortBackendMsg, DetokenizeMsg, ExitMsg, UserMsg
from ..reasoning import effective_reasoning_state
from ..utils.logger import init_logger
from .cache import CacheManager
from .config import SchedulerConfig
from .decode import DecodeManager
from .phase_policy import MixedPhaseFairPolicy
from .prefill import PendingReq, PrefillManager
from .stats import StatsTracker
from .table import TableManager

logger = init_logger(__name__)


def decide_max_sequence_admission(input_len: int, max_tokens: int, max_seq_len: int) -> Tuple[bool, int, str]:
    """(admit, clipped max_tokens, reason).  A prompt that leaves no room for one output token is rejected; an
    output budget that would pass the sequence limit is clipped (python/minisgl/scheduler/scheduler.py:62-122)."""
    if input_len <= 0:
        return False, 0, "empty prompt"
    if input_len >= max_seq_len:
        return False, 0, f"prompt of {input_len} tokens exceeds the maximum sequence length {max_seq_len}"
    return True, max(min(max_tokens, max_seq_len - input_len), 1), ""


@dataclass
class ForwardData:
    batch: Batch
    output: ForwardOutput
    epochs: List[Tuple[Req, int, int]]


class RequestAllFinished(Exception):
    pass


class Scheduler:
    def __init__(self, config: SchedulerConfig, engine: Optional[Engine] = None):
        self.config = config
        self.engine = engine or Engine(config)
        e = self.engine
        self.device, self.ps = e.device, e.page_size
        self.tp = config.tp_info
        self.table = TableManager(e.config.max_running_req)
        self.cache = CacheManager(e.pool, e.page_table, self.ps, e.model_config.window_size,
                                  enable_prefix_cache=config.cache_type == "radix")
        self.decode = DecodeManager(self.ps)
        self.prefill = PrefillManager(self.cache, self.table, self.decode, self.ps, e.max_seq_len)
        self.policy = MixedPhaseFairPolicy(isolated_prefill_budget=config.max_extend_tokens)
        self.stats = StatsTracker(config.stats_log_interval)
        self.eos_token_id = e.model_config.eos_token_id
        self.think_end_token_id = e.reasoning_token_ids.think_end if e.reasoning_token_ids else -1
        self.pending_retire: List[Req] = []
        self.finished_uids: set = set()
        self.io = None
        self.step_log: List[Dict[str, Any]] = []
        self.record_steps = False
        self.bytes_h2d = self.bytes_d2h = 0
        from ..env import ENV

        self.check_window = bool(ENV.DEBUG_BOUNDS)   # assert window residency before every forward
        self.heartbeat = None
        if getattr(config, "heartbeat_name", ""):
            from ..utils.heartbeat import HeartbeatBoard

            self.heartbeat = HeartbeatBoard(config.heartbeat_name, self.tp.size, create=False)

    def _beat(self, busy: bool) -> None:
        if self.heartbeat is not None:
            self.heartbeat.beat(self.tp.rank, busy)

    # ------------------------------------------------------------------ messages
    def _process_one_msg(self, msg) -> None:
        if isinstance(msg, UserMsg):
            ok, max_tokens, why = decide_max_sequence_admission(len(msg.input_ids), msg.sampling_params.max_tokens,
                                                                self.engine.max_seq_len)
            if not ok:
                logger.warning_rank0("request %d rejected: %s", msg.uid, why)
                self._reply(DetokenizeMsg(msg.uid, 0, True, "length_rejected"))
                return
            msg.sampling_params.max_tokens = max_tokens
            ids = msg.input_ids.to(torch.int32)
            self.prefill.add_one_req(PendingReq(msg.uid, ids, msg.sampling_params, msg.reasoning_effort))
        elif isinstance(msg, AbortBackendMsg):
            self._abort(msg.uid)
        elif isinstance(msg, ExitMsg):
            raise KeyboardInterrupt
        else:
            raise TypeError(f"unexpected backend message {type(msg).__name__}")

    def _abort(self, uid: int) -> None:
        if any(p.uid == uid for p in self.prefill.pending):
            # not admitted yet: nothing to release, but whoever collects results must learn that it ended
            self.prefill.abort(uid)
            self._on_reply(DetokenizeMsg(uid, 0, True, "abort"))
            return
        req = self.prefill.abort(uid)
        if req is None:
            req = next((r for r in self.decode.running if r.uid == uid), None)
        if req is not None and req.lifecycle.is_open:
            self.decode.remove(req)
            self._commit_terminal(req, "abort")

    def _reply(self, msg: DetokenizeMsg) -> None:
        if self.io is not None and self.tp.is_primary():
            self.io.send_result([msg])
        self._on_reply(msg)

    def _on_reply(self, msg: DetokenizeMsg) -> None:  # hook for the offline LLM
        pass

    # ------------------------------------------------------------------ scheduling
    def _schedule_next_batch(self) -> Optional[Tuple[Batch, BatchSamplingArgs]]:
        pre, dec = self.prefill.runnable, self.decode.runnable
        decision = self.policy.choose(prefill_runnable=pre, decode_runnable=dec)
        batch = None
        if decision.phase == "prefill":
            batch = self.prefill.schedule_next_batch(decision.prefill_budget)
            if batch is None and dec:
                batch = self._schedule_decode()
        elif decision.phase == "decode":
            batch = self._schedule_decode()
        self.policy.record_scheduled(batch.phase if batch else None, prefill_runnable=pre, decode_runnable=dec)
        if batch is None:
            return None
        return batch, self._prepare_batch(batch)

    def _schedule_decode(self) -> Optional[Batch]:
        """The decode batch of the running requests that have storage for their next position.  Admission reserves
        every page a request can need, so a failure here means the window-slot pool ran dry; the request that cannot
        continue is ended (``abort``), the others carry on, and the scheduling loop survives."""
        batch = self.decode.schedule_next_batch()
        if batch is None:
            return None
        keep = []
        for r in batch.reqs:
            if self.cache.try_allocate(r, r.device_len):
                keep.append(r)
            else:
                logger.warning_rank0("request %d ended: no KV storage for its next token (%s)", r.uid,
                                     self.cache.prefix_metrics_snapshot())
                self.decode.remove(r)
                self._commit_terminal(r, "abort")
        if not keep:
            return None
        batch.reqs = keep
        return batch

    def _prepare_batch(self, batch: Batch) -> BatchSamplingArgs:
        e, ps = self.engine, self.ps
        reqs = batch.reqs
        if self.check_window:
            for r, n in zip(reqs, batch.chunk_lens if batch.is_prefill else [1] * len(reqs)):
                self.cache.assert_window_resident(r, r.cached_len, r.cached_len + n - 1)
        if batch.is_decode:
            bs = len(reqs)
            padded = e.graph_runner.padded_size(bs) if e.graph_runner is not None else bs
            host = torch.zeros(4, padded, dtype=torch.int32, pin_memory=e.is_cuda)
            host[3, 0] = bs                       # number of valid rows, read by the captured graph
            pos = [r.device_len - 1 for r in reqs]
            host[0, :bs] = torch.tensor(pos, dtype=torch.int32)
            host[1, :bs] = torch.tensor([r.table_idx for r in reqs], dtype=torch.int32)
            host[2, :bs] = torch.tensor([r.pages[p // ps] * ps + p % ps for r, p in zip(reqs, pos)], dtype=torch.int32)
            if padded > bs:
                host[0, bs:] = 0
                host[1, bs:] = e.dummy_slot
                host[2, bs:] = e.pool.dummy_page * ps
            dev = host.to(self.device, non_blocking=True)
            self.bytes_h2d += host.numel() * 4
            batch.positions, batch.slots, batch.out_loc = dev[0], dev[1], dev[2]
            batch.device_block = dev
            batch.input_ids = None                # gathered on the device from the previous step's samples
            batch.last_idx = None
            batch.num_token_non_padded = bs
            batch.padded_reqs = list(reqs) + [None] * (padded - bs)
            batch.max_context = max(r.device_len for r in reqs)
        else:
            total = sum(batch.chunk_lens)
            host = torch.empty(4, total, dtype=torch.int32, pin_memory=e.is_cuda)
            last, o = [], 0
            for r, n in zip(reqs, batch.chunk_lens):
                a = r.cached_len
                host[0, o:o + n] = r.input_ids[a:a + n]
                host[1, o:o + n] = torch.arange(a, a + n, dtype=torch.int32)
                host[2, o:o + n] = r.table_idx
                pg = torch.tensor(r.pages, dtype=torch.int32)
                p = torch.arange(a, a + n)
                host[3, o:o + n] = pg[p // ps] * ps + (p % ps).to(torch.int32)
                o += n
                last.append(o - 1)
            dev = host.to(self.device, non_blocking=True)
            self.bytes_h2d += host.numel() * 4
            batch.input_ids, batch.positions, batch.slots, batch.out_loc = dev[0], dev[1], dev[2], dev[3]
            batch.last_idx = torch.tensor(last, dtype=torch.int64).to(self.device, non_blocking=True)
            batch.num_token_non_padded = total
            batch.padded_reqs = list(reqs)
            batch.max_context = max(r.cached_len + n for r, n in zip(reqs, batch.chunk_lens))
        if isinstance(e.sampler, ReasoningSampler):
            states = [int(r.reasoning_state) for r in reqs]
            return e.sampler.prepare(batch, states)
        return e.sampler.prepare(batch)

    def _forward(self, batch: Batch, args: BatchSamplingArgs) -> ForwardData:
        epochs = [(r, r.lifecycle.admission, r.lifecycle.launch()) for r in batch.reqs]
        if batch.is_prefill:
            finals = batch.is_final
            chunks = batch.chunk_lens
            saved = [(r.cached_len, r.device_len) for r in batch.reqs]
        out = self.engine.forward_batch(batch, args)
        if batch.is_prefill:
            # forward_batch advanced every request by one token; partial chunks advance by their chunk instead
            for r, (c0, d0), n, fin in zip(batch.reqs, saved, chunks, finals):
                if not fin:
                    r.cached_len, r.device_len = c0 + n, d0
            self.stats.on_prefill(sum(chunks))
            for r, fin in zip(batch.reqs, finals):
                if fin:
                    self.decode.add(r)
        else:
            self.stats.on_decode(batch.size)
            self.decode.filter_reqs(batch.reqs)
        self.bytes_d2h += out.next_tokens_cpu.numel() * out.next_tokens_cpu.element_size()
        if out.status is not None:
            self.bytes_d2h += 32   # the status word snapshot
        return ForwardData(batch, out, epochs)

    # ------------------------------------------------------------------ results
    def _process_last_data(self, last: Optional[ForwardData]) -> None:
        if last is None:
            return
        if last.output.copy_done_event is not None:
            last.output.copy_done_event.synchronize()
        if last.output.status is not None:
            # a kernel that gave up a wait (a peer GPU that stopped answering) left garbage behind: stop here, loudly.
            # The exception ends this scheduler process; the supervisor then turns the server to 503.
            last.output.status.check()
        batch, toks = last.batch, last.output.next_tokens_cpu
        finals = batch.is_final if batch.is_prefill else [True] * batch.size
        replies: List[DetokenizeMsg] = []
        for i, (req, gen, epoch) in enumerate(last.epochs):
            req.lifecycle.land(gen, epoch)
            if not req.lifecycle.is_open:
                continue  # aborted / finished while this forward was in flight
            if not finals[i]:
                self.cache.release_swa_behind(req)
                continue
            tok = int(toks[i])
            req.append_host(toks[i:i + 1])
            req.observe_generated_token(tok, think_end_token_id=self.think_end_token_id)
            done_eos = (not req.sampling_params.ignore_eos) and tok == self.eos_token_id
            done_len = not req.can_commit_token
            finished = done_eos or done_len
            reason = "stop" if done_eos else ("length" if done_len else None)
            # the first reply of a request (the one its last prefill chunk produces) carries the prompt length
            replies.append(DetokenizeMsg(req.uid, tok, finished, reason,
                                         req.prompt_len if batch.is_prefill else None))
            if batch.is_prefill:
                self.cache.cache_req(req, finished=False)
            self.cache.release_swa_behind(req)
            if finished:
                self.decode.remove(req)
                self._commit_terminal(req, reason, announce=False)
        if replies:
            if self.io is not None and self.tp.is_primary():
                self.io.send_result(replies)
            for m in replies:
                self._on_reply(m)
        self._retire_ready()

    def _commit_terminal(self, req: Req, reason: str, announce: bool = True) -> None:
        req.lifecycle.end(reason)
        self.pending_retire.append(req)
        self.finished_uids.add(req.uid)
        if announce:
            msg = DetokenizeMsg(req.uid, 0, True, reason)
            if reason != "abort":
                self._reply(msg)
            else:
                self._on_reply(msg)  # nobody waits for an aborted request online; the offline collector does
        self._retire_ready()

    def _retire_ready(self) -> None:
        """Resources go back only once every forward issued for the request has completed."""
        keep = []
        for req in self.pending_retire:
            if req.lifecycle.may_release:
                self.cache.cache_req(req, finished=True)
                self.table.free(req.table_idx)
                req.lifecycle.released()
            else:
                keep.append(req)
        self.pending_retire = keep

    # ------------------------------------------------------------------ loops
    def receive_msg(self, blocking: bool) -> List[Any]:
        if self.io is None:
            return []
        return self.io.receive_msg(blocking)

    def _idle(self) -> bool:
        return not (self.prefill.runnable or self.decode.runnable)

    def overlap_loop(self, last: Optional[ForwardData]) -> Optional[ForwardData]:
        blocking = self._idle() and last is None
        self._beat(busy=not blocking)  # an idle rank blocks in receive and is not expected to stamp
        for msg in self.receive_msg(blocking):
            self._process_one_msg(msg)
        if isinstance(self.engine.sampler, ReasoningSampler):
            # the structural-token mask depends on the previous sample: commit it before scheduling
            self._process_last_data(last)
            last = None
        nxt = self._schedule_next_batch()
        ongoing = None
        if nxt is not None:
            ongoing = self._forward(*nxt)
        self._process_last_data(last)
        self._log_stats()
        return ongoing

    def normal_loop(self) -> None:
        blocking = self._idle()
        self._beat(busy=not blocking)
        for msg in self.receive_msg(blocking):
            self._process_one_msg(msg)
        nxt = self._schedule_next_batch()
        if nxt is not None:
            self._process_last_data(self._forward(*nxt))
        self._log_stats()

    def run_forever(self) -> None:
        from ..env import ENV

        try:
            if ENV.DISABLE_OVERLAP_SCHEDULING.value:
                while True:
                    self.normal_loop()
            else:
                last = None
                while True:
                    last = self.overlap_loop(last)
        except KeyboardInterrupt:
            logger.info_rank0("scheduler exiting")

    def _log_stats(self) -> None:
        if self.config.disable_log_stats:
            return
        used = 1.0 - self.engine.pool.num_free_pages / max(self.engine.pool.sizes.num_pages, 1)
        line = self.stats.maybe_report(len(self.decode.running), len(self.prefill.pending) + len(self.prefill.resident),
                                       used)
        if line:
            logger.info_rank0(line)

    def sync_all_ranks(self) -> None:
        self.engine.sync_all_ranks()

    def shutdown(self) -> None:
        self.engine.shutdown()
