"""``python -m minisgl`` entry: parse arguments, start the API server, which spawns the backend processes
(one scheduler per tensor-parallel rank, a detokenizer, optional extra tokenizers) under a supervisor
(python/minisgl/server/launch.py:17-164 of the reference)."""
from __future__ import annotations

import dataclasses
import os
from typing import List

from ..parallel.info import DistributedInfo
from ..utils.logger import init_logger
from .args import ServerArgs, parse_args
from .supervisor import ProcessSpec, ServerProcessSupervisor

logger = init_logger(__name__)


def _run_scheduler(args: ServerArgs, ack_queue=None, role: str = "") -> None:
    """Child process body of one rank.  Built under no_grad (not inference_mode: weight tensors keep version
    counters, which the engine's caches key on)."""
    import torch

    from ..scheduler.io import SchedulerIO
    from ..scheduler.scheduler import Scheduler

    rank = args.tp_info.rank
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(args.tp_info.size))
    if args.silent_output:
        import logging

        logging.disable(logging.INFO)
    with torch.no_grad():
        sched = Scheduler(args)
        if args.enable_reasoning_sampler_contract:
            from ..reasoning import resolve_reasoning_token_ids
            from ..utils.hf import load_tokenizer

            ids = resolve_reasoning_token_ids(load_tokenizer(args.model_path))
            sched.engine.enable_reasoning_sampler(ids)
            sched.think_end_token_id = ids.think_end
        sched.io = SchedulerIO(args, sched.engine.cpu_group)
        sched.sync_all_ranks()
        if ack_queue is not None:
            ack_queue.put(role)
        try:
            sched.run_forever()
        finally:
            sched.io.stop()
            sched.shutdown()


def backend_specs(args: ServerArgs) -> List[ProcessSpec]:
    from ..tokenizer.server import tokenize_worker

    specs = []
    for r in range(args.tp_info.size):
        a = dataclasses.replace(args, tp_info=DistributedInfo(r, args.tp_info.size))
        specs.append(ProcessSpec(f"scheduler-{r}", _run_scheduler, {"args": a}, needs_ack=(r == 0)))
    common = dict(tokenizer_path=args.model_path, backend_addr=args.zmq_backend_addr,
                  frontend_addr=args.zmq_frontend_addr)
    specs.append(ProcessSpec("detokenizer", tokenize_worker,
                             dict(common, addr=args.zmq_detokenizer_addr, create=True, tokenizer_id=-1)))
    for i in range(args.num_tokenizer):
        specs.append(ProcessSpec(f"tokenizer-{i}", tokenize_worker,
                                 dict(common, addr=args.zmq_tokenizer_addr, create=(i == 0), tokenizer_id=i)))
    return specs


def start_server_processes(args: ServerArgs) -> ServerProcessSupervisor:
    from ..utils.heartbeat import HeartbeatBoard

    board = HeartbeatBoard(None, args.tp_info.size, create=True)  # the schedulers attach by name and stamp it
    args = dataclasses.replace(args, heartbeat_name=board.name)
    sup = ServerProcessSupervisor()
    sup.heartbeat = board
    sup.start(backend_specs(args))
    return sup


def graceful_exit_hook(args: ServerArgs):
    """Pushes ExitMsg to the backend (1 s send timeout / linger) so the schedulers leave their loops."""
    def hook():
        from ..message import ExitMsg
        from ..utils.mp import ZmqPushQueue

        q = ZmqPushQueue(args.zmq_backend_addr, create=False, send_timeout_ms=1000)
        try:
            q.put(ExitMsg())
        finally:
            q.stop()

    return hook


def launch_server(run_shell: bool = False) -> None:
    from .api_server import run_api_server

    args = parse_args(run_shell=run_shell)
    run_api_server(args, lambda: start_server_processes(args))
