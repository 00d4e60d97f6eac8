"""Process plumbing on CPU: the ZMQ queues, the scheduler's message distribution over two ranks (rank 0 pulls,
republishes and broadcasts the count; both ranks consume identical message lists; only rank 0 answers), and the local
tensor-parallel launcher (environment of the ranks, a failing rank ends its siblings)."""
import json
import os
import threading
import time
import uuid

import pytest
import torch

from io_worker import failing_rank, io_rank, ok_rank
from minisgl.core import SamplingParams
from minisgl.distributed.launch import launch_tensor_parallel
from minisgl.message import AbortBackendMsg, BatchBackendMsg, BatchTokenizerMsg, DetokenizeMsg, UserMsg
from minisgl.utils.mp import ZmqPubQueue, ZmqPullQueue, ZmqPushQueue, ZmqSubQueue


def _addr():
    return f"ipc:///tmp/minisgl_test_{uuid.uuid4().hex[:12]}"


def test_push_pull_and_pub_sub_round_trip():
    a = _addr()
    pull, push = ZmqPullQueue(a, create=True), ZmqPushQueue(a, create=False, send_timeout_ms=1000)
    assert pull.empty() and not pull.poll(10)
    msg = UserMsg(3, torch.arange(5, dtype=torch.int32), SamplingParams(max_tokens=7, temperature=0.5), "high")
    push.put(msg)
    assert pull.poll(2000)
    got = pull.get()
    assert isinstance(got, UserMsg) and got.uid == 3 and got.input_ids.tolist() == [0, 1, 2, 3, 4]
    assert got.sampling_params.max_tokens == 7 and got.reasoning_effort == "high"
    push.put(BatchBackendMsg(data=[AbortBackendMsg(4), AbortBackendMsg(5)]))
    raw = pull.get_raw()
    assert [m.uid for m in ZmqPullQueue.decode(raw).data] == [4, 5]
    b = _addr()
    pub, sub = ZmqPubQueue(b, create=True), ZmqSubQueue(b, create=False)
    deadline = time.time() + 5
    while sub.empty() and time.time() < deadline:       # a subscriber only sees what is published after it joined
        pub.put_raw(raw)
        time.sleep(0.05)
    assert [m.uid for m in sub.get().data] == [4, 5]
    for q in (pull, push, pub, sub):
        q.stop()


def test_two_ranks_consume_identical_messages_and_only_rank0_answers(tmp_path):
    suffix = "_t" + uuid.uuid4().hex[:10]
    out = str(tmp_path)
    detok = ZmqPullQueue(f"ipc:///tmp/minisgl_b200_detok{suffix}", create=True)

    def feeder():
        deadline = time.time() + 60
        while not os.path.exists(os.path.join(out, "ready")) and time.time() < deadline:
            time.sleep(0.05)
        push = ZmqPushQueue(f"ipc:///tmp/minisgl_b200_backend{suffix}", create=False, send_timeout_ms=2000)
        sp = SamplingParams(max_tokens=4)
        push.put(UserMsg(0, torch.arange(3, dtype=torch.int32), sp))
        time.sleep(0.2)
        push.put(BatchBackendMsg(data=[UserMsg(1, torch.arange(4, dtype=torch.int32), sp), AbortBackendMsg(0)]))
        push.put(UserMsg(2, torch.arange(2, dtype=torch.int32), sp))
        time.sleep(0.5)
        push.stop()

    th = threading.Thread(target=feeder, daemon=True)
    th.start()
    launch_tensor_parallel(2, io_rank, (out, suffix, 4), timeout_s=120)
    th.join(10)
    r0 = json.load(open(os.path.join(out, "rank0.json")))
    r1 = json.load(open(os.path.join(out, "rank1.json")))
    flat = lambda polls: [tuple(m) for p in polls for m in p]
    assert flat(r0) == flat(r1) == [("UserMsg", 0), ("UserMsg", 1), ("AbortBackendMsg", 0), ("UserMsg", 2)]
    assert r0 == r1                                      # and in the same polls: identical batches on every rank
    first = detok.get()
    assert isinstance(first, DetokenizeMsg) and (first.uid, first.next_token, first.finish_reason) == (7, 42, "length")
    second = detok.get()
    assert isinstance(second, BatchTokenizerMsg) and [m.uid for m in second.data] == [1, 2]
    assert detok.empty()                                  # rank 1 stayed silent
    detok.stop()


def test_launcher_sets_the_rank_environment(tmp_path):
    launch_tensor_parallel(2, ok_rank, (str(tmp_path),), timeout_s=60)
    assert sorted(f for f in os.listdir(tmp_path)) == ["ok0", "ok1"]
    assert open(tmp_path / "ok1").read() == "2 127.0.0.1"
    saved = dict(os.environ)
    try:
        launch_tensor_parallel(1, ok_rank, (str(tmp_path),))        # one rank runs in this very process
        assert open(tmp_path / "ok0").read() == "1 127.0.0.1"
    finally:
        os.environ.clear()
        os.environ.update(saved)
        from minisgl.parallel import info

        info._TP_INFO = None
    with pytest.raises(ValueError):
        launch_tensor_parallel(0, ok_rank, (str(tmp_path),))


def test_launcher_ends_the_siblings_of_a_failed_rank(tmp_path):
    t0 = time.time()
    with pytest.raises(RuntimeError, match="rank 1 failed with exit code 3"):
        launch_tensor_parallel(2, failing_rank, (str(tmp_path),), timeout_s=60)
    assert time.time() - t0 < 30                          # did not wait for the sleeping rank
