"""Collective communication for tensor parallelism.

Three interchangeable communicators (the model only sees ``all_reduce`` / ``all_gather_last``):

* ``NullComm``       single rank.
* ``TorchDistComm``  ``torch.distributed`` (NCCL on CUDA, gloo on CPU) -- the unfused baseline, and the path the
                     reference takes with ``--disable-pynccl`` (python/minisgl/distributed/impl.py:25-41).
* ``SymmComm``       (parallel/symm.py) in-kernel collectives over NVLink peer memory; the default on CUDA.  It
                     replaces the reference's PyNCCL symmetric-buffer all-reduce
                     (python/minisgl/kernel/csrc/src/pynccl.cu:73-176).

``init_distributed`` builds the control-plane (gloo) group and the data-plane communicator, one process per GPU.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..models.deepseek_v4 import Comm
from ..utils.logger import init_logger
from .info import DistributedInfo

logger = init_logger(__name__)


class NullComm(Comm):
    pass


class TorchDistComm(Comm):
    def __init__(self, info: DistributedInfo, group=None, vocab_size: Optional[int] = None):
        self.rank, self.size, self.group, self.vocab_size = info.rank, info.size, group, vocab_size
        self.counters = {"all_reduce": 0, "all_gather": 0}

    def all_reduce(self, x: torch.Tensor, tag: str = "") -> torch.Tensor:
        self.counters["all_reduce"] += 1
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x

    def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
        """[B, V/size] per rank -> [B, V] (rank-major along the last dim)."""
        self.counters["all_gather"] += 1
        b, vl = x.shape
        out = torch.empty(self.size * b, vl, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        full = out.view(self.size, b, vl).permute(1, 0, 2).reshape(b, self.size * vl)
        return full[:, : self.vocab_size] if self.vocab_size else full

    def barrier(self) -> None:
        dist.barrier(group=self.group)


def init_distributed(info: DistributedInfo, device: torch.device, addr: Optional[str] = None, timeout_s: float = 60.0,
                     fused: bool = True, vocab_size: Optional[int] = None, max_rows: int = 8192,
                     hidden: int = 4096) -> Tuple[Optional[object], Comm]:
    """Returns (cpu control group or None, communicator)."""
    if info.size == 1:
        return None, NullComm()
    timeout = datetime.timedelta(seconds=timeout_s)
    if not dist.is_initialized():
        init_method = addr or "env://"
        if init_method == "env://":
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
        backend = "cpu:gloo,cuda:nccl" if device.type == "cuda" else "gloo"
        kw = {"device_id": device} if device.type == "cuda" else {}
        dist.init_process_group(backend, init_method=init_method, rank=info.rank, world_size=info.size,
                                timeout=timeout, **kw)
    cpu_group = dist.new_group(backend="gloo", timeout=timeout)
    if device.type == "cuda" and fused:
        try:
            from .symm import SymmComm

            return cpu_group, SymmComm(info, device, vocab_size=vocab_size, max_rows=max_rows, hidden=hidden)
        except Exception as e:  # pragma: no cover - depends on the machine's NVLink setup
            logger.warning("fused NVLink collectives unavailable (%s); using torch.distributed", e)
    return cpu_group, TorchDistComm(info, None, vocab_size)
