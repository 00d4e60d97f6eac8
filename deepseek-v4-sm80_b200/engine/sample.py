"""Token sampling on top of the fused sampling kernel.

``Sampler.prepare`` turns the per-request ``SamplingParams`` of a batch into device tensors once per forward (or
into ``None`` when every request is greedy, in which case ``sample`` is a single argmax).  ``ReasoningSampler``
adds the DeepSeek-V4 structural-token contract: ``<think>`` is never sampled, EOS is masked while a request is
THINKING, ``</think>`` is masked otherwise.  Counterpart of python/minisgl/engine/sample.py:21-170 (which calls
flashinfer); here the masks ride along into one kernel (csrc/sampling.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..core import Batch
from ..ops import api as O
from ..reasoning import ReasoningState, ReasoningTokenIds
from ..utils.torch_utils import nvtx_annotate


@dataclass
class BatchSamplingArgs:
    temperature: Optional[torch.Tensor] = None   # fp32 [B]
    top_k: Optional[torch.Tensor] = None         # int32 [B]
    top_p: Optional[torch.Tensor] = None         # fp32 [B]
    uniform: Optional[torch.Tensor] = None       # fp32 [B]
    mask_ids: Optional[torch.Tensor] = None      # int32 [B, n]

    @property
    def all_greedy(self) -> bool:
        return self.temperature is None


def _to_dev(values, dtype, device):
    t = torch.tensor(values, dtype=dtype)
    if torch.device(device).type == "cuda":
        return t.pin_memory().to(device, non_blocking=True)
    return t


class Sampler:
    def __init__(self, device, vocab_size: int, seed: int = 0):
        self.device, self.vocab_size = device, vocab_size
        self.gen = torch.Generator()
        self.gen.manual_seed(seed)

    def prepare(self, batch: Batch) -> BatchSamplingArgs:
        reqs = batch.reqs
        if all(r.sampling_params.is_greedy for r in reqs):
            return BatchSamplingArgs()
        pad = batch.padded_size - len(reqs)
        temp = [0.0 if r.sampling_params.is_greedy else r.sampling_params.temperature for r in reqs] + [0.0] * pad
        top_k = [r.sampling_params.top_k for r in reqs] + [1] * pad
        top_p = [r.sampling_params.top_p for r in reqs] + [1.0] * pad
        u = torch.rand(len(temp), generator=self.gen).tolist()
        return BatchSamplingArgs(_to_dev(temp, torch.float32, self.device), _to_dev(top_k, torch.int32, self.device),
                                 _to_dev(top_p, torch.float32, self.device), _to_dev(u, torch.float32, self.device))

    @nvtx_annotate("Sampler")
    def sample(self, logits: torch.Tensor, args: BatchSamplingArgs) -> torch.Tensor:
        if args.all_greedy and args.mask_ids is None:
            return O.argmax(logits)
        b = logits.shape[0]
        dev = logits.device
        temp = args.temperature if args.temperature is not None else torch.zeros(b, dtype=torch.float32, device=dev)
        top_k = args.top_k if args.top_k is not None else torch.full((b,), -1, dtype=torch.int32, device=dev)
        top_p = args.top_p if args.top_p is not None else torch.ones(b, dtype=torch.float32, device=dev)
        u = args.uniform if args.uniform is not None else torch.full((b,), 0.5, dtype=torch.float32, device=dev)
        return O.sample(logits, temp[:b], top_k[:b], top_p[:b], u[:b], args.mask_ids)


class ReasoningSampler(Sampler):
    """Masks structural tokens according to each request's reasoning state before sampling."""

    def __init__(self, device, vocab_size: int, token_ids: ReasoningTokenIds, seed: int = 0):
        super().__init__(device, vocab_size, seed)
        self.token_ids = token_ids

    def mask_rows(self, states: List[int]) -> List[List[int]]:
        t = self.token_ids
        rows = []
        for s in states:
            second = t.eos if s == ReasoningState.THINKING else t.think_end
            rows.append([t.think_start, second])
        return rows

    def prepare(self, batch: Batch, states: Optional[List[int]] = None) -> BatchSamplingArgs:
        args = super().prepare(batch)
        if states is None:
            states = [int(r.reasoning_state) for r in batch.reqs]
        pad = batch.padded_size - len(states)
        rows = self.mask_rows(list(states) + [int(ReasoningState.CHAT)] * pad)
        args.mask_ids = _to_dev(rows, torch.int32, self.device)
        return args
