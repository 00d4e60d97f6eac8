"""Message plumbing of the online scheduler.

Rank 0 pulls tokenised requests from the tokenizer workers and republishes the raw bytes to the other ranks; every
loop iteration it also broadcasts, over the gloo control group, how many messages it took, so that all ranks consume
exactly the same set and build identical batches.  Only rank 0 sends results to the detokenizer.
(python/minisgl/scheduler/io.py:15-133 of the reference.)
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional

import torch

from ..message import BatchBackendMsg, BatchTokenizerMsg, DetokenizeMsg
from ..utils.mp import ZmqPubQueue, ZmqPullQueue, ZmqPushQueue, ZmqSubQueue
from .config import SchedulerConfig


def _flatten(msg) -> List[Any]:
    return list(msg.data) if isinstance(msg, BatchBackendMsg) else [msg]


class SchedulerIO:
    def __init__(self, config: SchedulerConfig, cpu_group, on_idle: Optional[Callable[[], None]] = None):
        self.tp, self.group, self.on_idle = config.tp_info, cpu_group, on_idle or (lambda: None)
        self.pull = self.push = self.pub = self.sub = None
        if self.tp.is_primary():
            self.pull = ZmqPullQueue(config.zmq_backend_addr, create=True)
            self.push = ZmqPushQueue(config.zmq_detokenizer_addr, create=False, send_timeout_ms=1000)
            if self.tp.size > 1:
                self.pub = ZmqPubQueue(config.zmq_scheduler_broadcast_addr, create=True)
        else:
            self.sub = ZmqSubQueue(config.zmq_scheduler_broadcast_addr, create=False)

    # ------------------------------------------------------------------ receive
    def receive_msg(self, blocking: bool = False) -> List[Any]:
        if self.tp.size == 1:
            return self._recv_single(blocking)
        return self._recv_rank0(blocking) if self.tp.is_primary() else self._recv_other(blocking)

    def _recv_single(self, blocking: bool) -> List[Any]:
        out: List[Any] = []
        if blocking:
            self.on_idle()
            out += _flatten(self.pull.get())
        while not self.pull.empty():
            out += _flatten(self.pull.get())
        return out

    def _bcast_count(self, n: int) -> int:
        import torch.distributed as dist

        t = torch.tensor([n], dtype=torch.int64)
        dist.broadcast(t, src=0, group=self.group)
        return int(t[0])

    def _recv_rank0(self, blocking: bool) -> List[Any]:
        raws: List[bytes] = []
        if blocking:
            self.on_idle()
            raws.append(self.pull.get_raw())
        while not self.pull.empty():
            raws.append(self.pull.get_raw())
        self._bcast_count(len(raws))
        out: List[Any] = []
        for raw in raws:
            self.pub.put_raw(raw)
            out += _flatten(ZmqPullQueue.decode(raw))
        return out

    def _recv_other(self, blocking: bool) -> List[Any]:
        if blocking:
            self.on_idle()
        n = self._bcast_count(-1)
        out: List[Any] = []
        for _ in range(n):
            out += _flatten(self.sub.get())
        return out

    # ------------------------------------------------------------------ send
    def send_result(self, replies: List[DetokenizeMsg]) -> None:
        if not self.tp.is_primary() or not replies:
            return
        self.push.put(replies[0] if len(replies) == 1 else BatchTokenizerMsg(data=list(replies)))

    def stop(self) -> None:
        for q in (self.pull, self.push, self.pub, self.sub):
            if q is not None:
                q.stop()
