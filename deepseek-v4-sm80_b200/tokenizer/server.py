"""Tokenizer / detokenizer worker process.

Loop: pull a (batch of) message(s); ``DetokenizeMsg`` -> incremental text -> ``UserReply`` to the API frontend;
``TokenizeMsg`` -> token ids -> ``UserMsg`` to scheduler rank 0; ``AbortMsg`` -> ``AbortBackendMsg``.
(python/minisgl/tokenizer/server.py:31-118 of the reference.)
"""
from __future__ import annotations

from typing import Any, List

from ..message import (AbortBackendMsg, AbortMsg, BatchBackendMsg, BatchFrontendMsg, BatchTokenizerMsg, DetokenizeMsg,
                       TokenizeMsg, UserMsg, UserReply)
from ..utils.logger import init_logger
from ..utils.mp import ZmqPullQueue, ZmqPushQueue

logger = init_logger(__name__)


def _unwrap(msg) -> List[Any]:
    return list(msg.data) if isinstance(msg, BatchTokenizerMsg) else [msg]


def handle_batch(msgs: List[Any], tokenize_mgr, detokenize_mgr, counts) -> tuple:
    """Pure step of the worker: returns (messages for the backend, replies for the frontend)."""
    detok = [m for m in msgs if isinstance(m, DetokenizeMsg)]
    tok = [m for m in msgs if isinstance(m, TokenizeMsg)]
    aborts = [m for m in msgs if isinstance(m, AbortMsg)]
    to_backend: List[Any] = []
    to_frontend: List[Any] = []
    if detok:
        texts = detokenize_mgr.detokenize(detok)
        for m, t in zip(detok, texts):
            n = counts.get(m.uid, 0) + (0 if m.finish_reason in ("length_rejected", "abort") else 1)
            counts[m.uid] = n
            to_frontend.append(UserReply(m.uid, t, m.finished, m.finish_reason, n, m.prompt_tokens))
            if m.finished:
                counts.pop(m.uid, None)
    if tok:
        ids = tokenize_mgr.tokenize(tok)
        for m, t in zip(tok, ids):
            to_backend.append(UserMsg(m.uid, t, m.sampling_params, m.reasoning_effort))
    for m in aborts:
        to_backend.append(AbortBackendMsg(m.uid))
    return to_backend, to_frontend


def tokenize_worker(*, tokenizer_path: str, addr: str, create: bool, backend_addr: str, frontend_addr: str,
                    local_bs: int = 1, tokenizer_id: int = -1, ack_queue=None, role: str = "tokenizer") -> None:
    from ..utils.hf import load_tokenizer
    from .detokenize import DetokenizeManager
    from .tokenize import TokenizeManager

    import signal

    def _terminate(signum, frame):  # the supervisor ends this worker with SIGTERM: leave through the finally below
        raise KeyboardInterrupt

    signal.signal(signal.SIGTERM, _terminate)
    tokenizer = load_tokenizer(tokenizer_path)
    tok_mgr, detok_mgr = TokenizeManager(tokenizer, tokenizer_path), DetokenizeManager(tokenizer)
    recv = ZmqPullQueue(addr, create=create)
    to_backend = ZmqPushQueue(backend_addr, create=False, send_timeout_ms=1000)
    to_frontend = ZmqPushQueue(frontend_addr, create=False, send_timeout_ms=1000)
    if ack_queue is not None:
        ack_queue.put(role)
    counts: dict = {}
    try:
        while True:
            msgs = _unwrap(recv.get())
            while len(msgs) < local_bs and not recv.empty():
                msgs += _unwrap(recv.get())
            if any(type(m).__name__ == "ExitMsg" for m in msgs):
                break
            b, f = handle_batch(msgs, tok_mgr, detok_mgr, counts)
            if b:
                to_backend.put(b[0] if len(b) == 1 else BatchBackendMsg(b))
            if f:
                to_frontend.put(f[0] if len(f) == 1 else BatchFrontendMsg(f))
    except KeyboardInterrupt:
        pass
    finally:
        for q in (recv, to_backend, to_frontend):
            q.stop()
