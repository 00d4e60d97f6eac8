"""Lifecycle of the server's child processes (one scheduler per rank, tokenizer / detokenizer workers).

* roles are unique; every child puts its role on a shared queue when it is ready; start-up fails if a child exits
  before acknowledging or if the acknowledgements do not arrive within the timeout (15 minutes by default: loading
  and graph capture of a large model take minutes);
* ``unexpected_exit`` reports a child that died while serving -- the API frontend polls it and turns the whole
  backend unavailable;
* ``shutdown`` is idempotent: optional graceful hook, then terminate, then kill, and it verifies every child was reaped.
Counterpart of python/minisgl/server/supervisor.py:16-208 of the reference.
"""
from __future__ import annotations

import multiprocessing as mp
import queue
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..utils.logger import init_logger

logger = init_logger(__name__)

STARTUP_TIMEOUT_S = 15 * 60.0


class SupervisorError(RuntimeError):
    pass


@dataclass
class ProcessSpec:
    role: str
    target: Callable[..., None]
    kwargs: Dict[str, Any] = field(default_factory=dict)
    needs_ack: bool = True


class ServerProcessSupervisor:
    def __init__(self, startup_timeout_s: float = STARTUP_TIMEOUT_S, poll_s: float = 0.1, mp_context: str = "spawn"):
        self.ctx = mp.get_context(mp_context)
        self.ack_queue = self.ctx.Queue()
        self.startup_timeout_s, self.poll_s = startup_timeout_s, poll_s
        self.children: Dict[str, Any] = {}
        self.started = False
        self.shut_down = False

    # ------------------------------------------------------------------ start
    def start(self, specs: List[ProcessSpec]) -> None:
        if self.started:
            raise SupervisorError("supervisor already started")
        roles = [s.role for s in specs]
        if len(set(roles)) != len(roles):
            raise SupervisorError(f"process roles must be unique: {roles}")
        self.started = True
        for s in specs:
            kw = dict(s.kwargs)
            kw.setdefault("ack_queue", self.ack_queue)
            kw.setdefault("role", s.role)
            p = self.ctx.Process(target=s.target, kwargs=kw, name=s.role, daemon=False)
            p.start()
            self.children[s.role] = p
        try:
            self._wait_for_readiness({s.role for s in specs if s.needs_ack})
        except BaseException:
            self.shutdown()
            raise

    def _wait_for_readiness(self, pending: set) -> None:
        deadline = time.monotonic() + self.startup_timeout_s
        while pending:
            try:
                role = self.ack_queue.get(timeout=self.poll_s)
                pending.discard(role)
                continue
            except queue.Empty:
                pass
            dead = self.unexpected_exit()
            if dead is not None:
                raise SupervisorError(f"child {dead[0]!r} exited with code {dead[1]} before it was ready")
            if time.monotonic() > deadline:
                raise SupervisorError(f"children not ready after {self.startup_timeout_s:.0f} s: {sorted(pending)}")

    # ------------------------------------------------------------------ runtime
    def unexpected_exit(self) -> Optional[Tuple[str, int]]:
        if self.shut_down:
            return None
        for role, p in self.children.items():
            if p.exitcode is not None:
                return role, p.exitcode
        return None

    def alive_roles(self) -> List[str]:
        return [r for r, p in self.children.items() if p.exitcode is None]

    # ------------------------------------------------------------------ stop
    def shutdown(self, graceful: Optional[Callable[[], None]] = None, grace_s: float = 5.0) -> None:
        if self.shut_down:
            return
        self.shut_down = True
        board = getattr(self, "heartbeat", None)
        if board is not None:
            board.close()
        if graceful is not None:
            try:
                graceful()
            except Exception as e:  # pragma: no cover
                logger.warning("graceful shutdown hook failed: %s", e)
            self._join_all(grace_s)
        for p in self.children.values():
            if p.exitcode is None:
                p.terminate()
        self._join_all(grace_s)
        for p in self.children.values():
            if p.exitcode is None:
                p.kill()
        self._join_all(grace_s)
        left = [r for r, p in self.children.items() if p.exitcode is None]
        if left:
            raise SupervisorError(f"children could not be reaped: {left}")

    def _join_all(self, timeout_s: float) -> None:
        deadline = time.monotonic() + timeout_s
        for p in self.children.values():
            p.join(max(deadline - time.monotonic(), 0.0))
