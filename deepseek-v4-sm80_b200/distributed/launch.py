"""Local tensor-parallel launcher: runs ``fn`` in N spawned processes with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*
set, polls them, and terminates the siblings as soon as one exits non-zero
(python/minisgl/distributed/launch.py:11-89 of the reference)."""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
import time
from typing import Any, Callable, Tuple


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank: int, world: int, port: int, fn: Callable, args: Tuple[Any, ...]) -> None:
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from ..parallel.info import set_tp_info

    set_tp_info(rank, world)
    fn(*args)


def launch_tensor_parallel(world_size: int, fn: Callable, args: Tuple[Any, ...] = (), poll_s: float = 0.2,
                           timeout_s: float | None = None) -> None:
    """Blocks until every rank exited 0; raises RuntimeError (after terminating the others) if one failed."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if world_size == 1:
        _entry(0, 1, _free_port(), fn, args)
        return
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn, args), name=f"tp-rank-{r}")
             for r in range(world_size)]
    for p in procs:
        p.start()
    t0 = time.monotonic()
    failed = None
    try:
        while True:
            alive = False
            for r, p in enumerate(procs):
                if p.exitcode is None:
                    alive = True
                elif p.exitcode != 0 and failed is None:
                    failed = (r, p.exitcode)
            if failed is not None or not alive:
                break
            if timeout_s is not None and time.monotonic() - t0 > timeout_s:
                failed = (-1, "timeout")
                break
            time.sleep(poll_s)
    finally:
        for p in procs:
            if p.exitcode is None:
                p.terminate()
        for p in procs:
            p.join(5)
    if failed is not None:
        raise RuntimeError(f"tensor-parallel rank {failed[0]} failed with exit code {failed[1]}; siblings terminated")
