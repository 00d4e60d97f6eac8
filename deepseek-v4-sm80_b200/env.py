"""Typed environment variables, prefix ``MINISGL_`` (python/minisgl/env.py:57-87 of the reference)."""
from __future__ import annotations

import os
from typing import Callable, Generic, Optional, TypeVar

T = TypeVar("T")


class EnvVar(Generic[T]):
    def __init__(self, name: str, default: T, parse: Callable[[str], T]):
        self.name, self.default, self.parse = "MINISGL_" + name, default, parse

    @property
    def value(self) -> T:
        raw = os.environ.get(self.name)
        if raw is None or raw == "":
            return self.default
        return self.parse(raw)

    def __bool__(self):
        return bool(self.value)


def _bool(s: str) -> bool:
    return s.strip().lower() in ("1", "true", "yes", "on")


def _mem(s: str) -> int:
    s = s.strip().upper()
    for suf, mul in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
        if s.endswith(suf):
            return int(float(s[:-1]) * mul)
    return int(s)


class _Env:
    SHELL_MAX_TOKENS = EnvVar("SHELL_MAX_TOKENS", 2048, int)
    SHELL_TOP_K = EnvVar("SHELL_TOP_K", -1, int)
    SHELL_TOP_P = EnvVar("SHELL_TOP_P", 1.0, float)
    SHELL_TEMPERATURE = EnvVar("SHELL_TEMPERATURE", 0.6, float)
    DISABLE_OVERLAP_SCHEDULING = EnvVar("DISABLE_OVERLAP_SCHEDULING", False, _bool)
    COMM_MAX_BUFFER_SIZE = EnvVar("PYNCCL_MAX_BUFFER_SIZE", 32 << 20, _mem)
    DISABLE_FUSED_COMM = EnvVar("DISABLE_FUSED_COMM", False, _bool)
    DISABLE_MULTIMEM = EnvVar("DISABLE_MULTIMEM", False, _bool)
    NVTX = EnvVar("NVTX", False, _bool)
    DEBUG_BOUNDS = EnvVar("DEBUG_BOUNDS", False, _bool)
    DUMMY_WEIGHT_ON_HOST = EnvVar("DUMMY_WEIGHT_ON_HOST", False, _bool)   # draw random weights on the CPU, copy shards
    PEER_WAIT_MS = EnvVar("PEER_WAIT_MS", 2000, int)      # limit of in-kernel waits on other GPUs
    DISABLE_STATUS_CHECK = EnvVar("DISABLE_STATUS_CHECK", False, _bool)   # per-step device status read


ENV = _Env()
