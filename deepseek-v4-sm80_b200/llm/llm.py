"""Offline API: ``LLM(model).generate(prompts, sampling_params)``.

A ``Scheduler`` subclass in offline mode: requests are fed from a local list (up to the prefill budget per poll),
results are collected instead of being sent to a detokenizer, and the loop ends when every request has finished
(python/minisgl/llm/llm.py:35-187 of the reference).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..core import SamplingParams
from ..message import DetokenizeMsg, UserMsg
from ..parallel.info import DistributedInfo, try_get_tp_info
from ..scheduler.config import SchedulerConfig
from ..scheduler.scheduler import RequestAllFinished, Scheduler


@dataclass
class RequestOutput:
    uid: int
    token_ids: List[int] = field(default_factory=list)
    text: Optional[str] = None
    finish_reason: Optional[str] = None
    t_first: Optional[float] = None
    t_tokens: List[float] = field(default_factory=list)


class LLM(Scheduler):
    def __init__(self, model_path: str = "", dtype: torch.dtype = torch.bfloat16, **kwargs):
        info = kwargs.pop("tp_info", None) or try_get_tp_info() or self._info_from_env()
        config = SchedulerConfig(model_path=model_path, tp_info=info, dtype=dtype, offline_mode=True, **kwargs)
        super().__init__(config)
        self.tokenizer = None
        if model_path:
            try:
                from ..utils.hf import load_tokenizer

                self.tokenizer = load_tokenizer(model_path)
            except Exception:
                self.tokenizer = None
        self._queue: List[UserMsg] = []
        self._results: Dict[int, RequestOutput] = {}
        self._next_uid = 0
        self._open = 0
        self._gap = 0          # engine steps between two released requests (0: release by prefill budget)
        self._since = 0

    @property
    def phase_steps(self) -> Dict[str, int]:
        """Engine forwards so far, per phase (for scenario harnesses)."""
        return {"prefill": self.stats.prefill_steps, "decode": self.stats.decode_steps}

    @staticmethod
    def _info_from_env() -> DistributedInfo:
        import os

        return DistributedInfo(int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))

    # offline message source: release queued requests as the prefill budget allows
    def receive_msg(self, blocking: bool) -> List[Any]:
        if not self._queue:
            if self._open == 0:
                raise RequestAllFinished()
            return []
        if self._gap > 0:  # staggered arrival: one request every `gap` polls
            self._since += 1
            if self._since < self._gap and self._open_released > 0:
                return []
            self._since = 0
            self._open_released += 1
            return [self._queue.pop(0)]
        budget, out = self.config.max_extend_tokens, []
        while self._queue and (budget > 0 or not out):
            m = self._queue.pop(0)
            budget -= len(m.input_ids)
            out.append(m)
        return out

    def _on_reply(self, msg: DetokenizeMsg) -> None:
        r = self._results.get(msg.uid)
        if r is None or r.finish_reason is not None:
            return
        now = time.perf_counter()
        if msg.finish_reason != "length_rejected" and not (msg.finished and msg.finish_reason == "abort"):
            r.token_ids.append(msg.next_token)
            r.t_tokens.append(now)
            if r.t_first is None:
                r.t_first = now
        if msg.finished:
            r.finish_reason = msg.finish_reason
            self._open -= 1

    def abort(self, uid: int) -> None:
        """Ends request ``uid`` wherever it is: still queued here, waiting for admission, prefilling or decoding.  Its
        RequestOutput keeps the tokens produced so far and gets finish_reason ``abort``."""
        for m in self._queue:
            if m.uid == uid:
                self._queue.remove(m)
                self._on_reply(DetokenizeMsg(uid, 0, True, "abort"))
                return
        self._abort(uid)

    def _encode(self, prompt, reasoning_effort) -> torch.Tensor:
        if isinstance(prompt, torch.Tensor):
            return prompt.to(torch.int32).cpu()
        if isinstance(prompt, (list, tuple)) and (not prompt or isinstance(prompt[0], int)):
            return torch.tensor(list(prompt), dtype=torch.int32)
        if self.tokenizer is None:
            raise ValueError("text prompts need a tokenizer (model_path with tokenizer files)")
        if isinstance(prompt, str):
            return torch.tensor(self.tokenizer.encode(prompt), dtype=torch.int32)
        from ..tokenizer.tokenize import TokenizeManager

        return TokenizeManager(self.tokenizer, self.config.model_path).encode_messages(prompt, reasoning_effort)

    def generate(self, prompts: Sequence[Any], sampling_params: Union[SamplingParams, Sequence[SamplingParams]],
                 reasoning_effort: Optional[str] = None, arrival_gap_steps: int = 0) -> List[RequestOutput]:
        """prompts: token-id lists / tensors, strings, or chat message lists.  Returns one RequestOutput per prompt
        (token ids, decoded text when a tokenizer is available, finish reason, per-token host timestamps).
        ``arrival_gap_steps`` > 0 releases one request every that many scheduler polls instead of all at once."""
        self._gap, self._since, self._open_released = int(arrival_gap_steps), 0, 0
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        uids = []
        self.t_submit = time.perf_counter()
        for p, sp in zip(prompts, sampling_params):
            uid = self._next_uid
            self._next_uid += 1
            ids = self._encode(p, reasoning_effort)
            self._queue.append(UserMsg(uid, ids, SamplingParams(**vars(sp)), reasoning_effort))
            self._results[uid] = RequestOutput(uid)
            self._open += 1
            uids.append(uid)
        try:
            last = None
            while True:
                last = self.overlap_loop(last)
        except RequestAllFinished:
            pass
        outs = [self._results.pop(u) for u in uids]
        if self.tokenizer is not None:
            for o in outs:
                o.text = self.tokenizer.decode(o.token_ids)
        return outs
