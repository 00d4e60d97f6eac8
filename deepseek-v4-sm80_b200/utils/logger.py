"""Coloured, rank-aware logging: ``[date|time|pid|core|rank=N]`` with ``LOG_LEVEL`` / ``LOG_PID`` from the environment
(same surface as python/minisgl/utils/logger.py:9-128 of the reference)."""
from __future__ import annotations

import logging
import os
import sys

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[35m"}
_RANK = {"rank": None}


def set_log_rank(rank: int) -> None:
    _RANK["rank"] = rank


class _Fmt(logging.Formatter):
    def format(self, record):
        pid = f"|{os.getpid()}" if os.environ.get("LOG_PID") else ""
        rank = f"|rank={_RANK['rank']}" if _RANK["rank"] is not None else ""
        color = _COLORS.get(record.levelname, "") if sys.stderr.isatty() else ""
        reset = "\033[0m" if color else ""
        head = f"[{self.formatTime(record, '%Y-%m-%d|%H:%M:%S')}{pid}|{record.name}{rank}]"
        return f"{color}{head} {record.levelname}{reset} {record.getMessage()}"


class _Logger(logging.Logger):
    def info_rank0(self, msg, *a, **k):
        if not _RANK["rank"]:
            self.info(msg, *a, **k)

    def warning_rank0(self, msg, *a, **k):
        if not _RANK["rank"]:
            self.warning(msg, *a, **k)

    def debug_rank0(self, msg, *a, **k):
        if not _RANK["rank"]:
            self.debug(msg, *a, **k)


logging.setLoggerClass(_Logger)


def init_logger(name: str, level=None) -> _Logger:
    lg = logging.getLogger(name)
    if not lg.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(_Fmt())
        lg.addHandler(h)
        lg.propagate = False
    lg.setLevel(level or os.environ.get("LOG_LEVEL", "INFO").upper())
    return lg  # type: ignore[return-value]
