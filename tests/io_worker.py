"""Rank body for the scheduler-IO test (run by launch_tensor_parallel): every rank builds a SchedulerIO over a gloo
group, rank 0's feeder pushes request batches into the backend socket, and each rank writes the uids it consumed per
poll into its own file."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def io_rank(out_dir: str, suffix: str, expect: int) -> None:
    import torch.distributed as dist

    from minisgl.parallel.info import DistributedInfo
    from minisgl.scheduler.config import SchedulerConfig
    from minisgl.scheduler.io import SchedulerIO

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = SchedulerConfig(model_path="", tp_info=DistributedInfo(rank, world), offline_mode=False,
                          _unique_suffix=suffix)
    idle = []
    io = SchedulerIO(cfg, dist.group.WORLD, on_idle=lambda: idle.append(1))
    dist.barrier()            # every subscriber is connected before rank 0 is fed
    time.sleep(0.3)
    if rank == 0:
        open(os.path.join(out_dir, "ready"), "w").write("1")
    polls, seen = [], 0
    deadline = time.time() + 60
    while seen < expect and time.time() < deadline:
        msgs = io.receive_msg(blocking=False)
        if msgs:
            polls.append([(type(m).__name__, m.uid) for m in msgs])
            seen += len(msgs)
        else:
            time.sleep(0.01)
    if rank == 0:
        from minisgl.message import DetokenizeMsg

        io.send_result([DetokenizeMsg(7, 42, True, "length")])
        io.send_result([DetokenizeMsg(1, 5, False), DetokenizeMsg(2, 6, False)])
    else:
        from minisgl.message import DetokenizeMsg

        io.send_result([DetokenizeMsg(9, 9, True, "stop")])   # only rank 0 answers: this must be a no-op
    json.dump(polls, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    dist.barrier()
    io.stop()
    dist.destroy_process_group()


def ok_rank(out_dir: str) -> None:
    rank = os.environ["RANK"]
    open(os.path.join(out_dir, f"ok{rank}"), "w").write(os.environ["WORLD_SIZE"] + " " + os.environ["MASTER_ADDR"])


def failing_rank(out_dir: str) -> None:
    if os.environ["RANK"] == "1":
        sys.exit(3)
    time.sleep(60)            # the launcher must not wait for this one
