"""HTTP contract of the OpenAI-compatible frontend against an in-process fake frontend, argument parsing, the process
supervisor (real child processes that acknowledge, exit early or hang) and message serialisation."""
import asyncio
import json
import multiprocessing as mp
import time

import pytest
import torch
from fastapi.testclient import TestClient

from minisgl.core import SamplingParams
from minisgl.message import (AbortBackendMsg, BatchBackendMsg, DetokenizeMsg, ExitMsg, TokenizeMsg, UserMsg, UserReply,
                             pack, unpack)
from minisgl.server.api_server import (BackendUnavailable, ReasoningContentParser, ServeInfo, create_app)
from minisgl.server.args import parse_args
from minisgl.server.supervisor import ProcessSpec, ServerProcessSupervisor, SupervisorError
from minisgl.utils.misc import UNSET


class FakeFrontend:
    def __init__(self, pieces, finish="stop"):
        self.pieces, self.finish, self.available, self.unavailable_reason = pieces, finish, True, None
        self.submitted, self.aborted = [], []

    async def submit(self, text, sampling, effort):
        if not self.available:
            raise BackendUnavailable("down")
        self.submitted.append((text, sampling, effort))
        return len(self.submitted) - 1

    async def stream(self, uid):
        for i, p in enumerate(self.pieces):
            last = i == len(self.pieces) - 1
            yield UserReply(uid, p, last, self.finish if last else None, i + 1)

    async def abort(self, uid):
        self.aborted.append(uid)


def client(pieces, finish="stop"):
    fe = FakeFrontend(pieces, finish)
    return TestClient(create_app(fe, ServeInfo(("dsv4", "/models/dsv4"), "/models/dsv4"))), fe


BODY = {"model": "dsv4", "messages": [{"role": "user", "content": "hi"}]}


def test_chat_completion_non_stream_and_usage():
    c, fe = client(["Hel", "lo"], "length")
    r = c.post("/v1/chat/completions", json=dict(BODY, max_tokens=5, temperature=0))
    assert r.status_code == 200
    j = r.json()
    assert j["object"] == "chat.completion" and j["choices"][0]["message"] == {"role": "assistant", "content": "Hello"}
    assert j["choices"][0]["finish_reason"] == "length" and j["usage"]["completion_tokens"] == 2
    text, sp, effort = fe.submitted[0]
    assert text == [{"role": "user", "content": "hi"}] and sp.max_tokens == 5 and sp.is_greedy and effort is None


def test_defaults_and_max_completion_tokens_precedence():
    c, fe = client(["x"])
    c.post("/v1/chat/completions", json=dict(BODY, max_tokens=7, max_completion_tokens=3))
    c.post("/v1/chat/completions", json=BODY)
    assert fe.submitted[0][1].max_tokens == 3
    assert fe.submitted[1][1].max_tokens == 2048 and fe.submitted[1][1].temperature == 1.0


def test_streaming_chunks_reasoning_split_and_done():
    c, fe = client(["think</th", "ink>ans", "wer"])
    body = dict(BODY, stream=True, reasoning_effort="high", stream_options={"include_usage": True})
    with c.stream("POST", "/v1/chat/completions", json=body) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    reasoning = "".join(ch["choices"][0]["delta"].get("reasoning_content", "") for ch in chunks if ch["choices"])
    content = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks if ch["choices"])
    assert reasoning == "think" and content == "answer"
    assert chunks[-2]["choices"][0]["finish_reason"] == "stop" and chunks[-2]["choices"][0]["delta"] == {}
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 3
    assert fe.submitted[0][2] == "high"


@pytest.mark.parametrize("extra,param,status", [
    ({"tools": []}, "tools", 400), ({"logprobs": True}, "logprobs", 400), ({"n": 2}, "n", 400),
    ({"stop": ["x"]}, "stop", 400), ({"presence_penalty": 0.5}, "presence_penalty", 400), ({"seed": 1}, "seed", 400),
    ({"temperature": -1}, "temperature", 400), ({"top_k": 0}, "top_k", 400), ({"top_p": 1.5}, "top_p", 400),
    ({"bogus_field": 1}, "bogus_field", 400), ({"prompt": "x"}, "prompt", 400), ({"response_format": {}}, "response_format", 400),
    ({"reasoning_effort": "low"}, "reasoning_effort", 400),
])
def test_unsupported_parameters_are_rejected_with_openai_errors(extra, param, status):
    c, fe = client(["x"])
    r = c.post("/v1/chat/completions", json=dict(BODY, **extra))
    assert r.status_code == status
    err = r.json()["error"]
    assert err["type"] == "invalid_request_error" and err["param"] == param and err["message"]
    assert not fe.submitted


def test_model_name_check_models_route_and_v1_root():
    c, _ = client(["x"])
    r = c.post("/v1/chat/completions", json=dict(BODY, model="other"))
    assert r.status_code == 404 and r.json()["error"]["code"] == "model_not_found"
    assert c.post("/v1/chat/completions", json=dict(BODY, model="/models/dsv4")).status_code == 200
    m = c.get("/v1/models").json()["data"][0]
    assert m == {"id": "dsv4", "object": "model", "created": 0, "owned_by": "mini-sglang", "root": "/models/dsv4"}
    for method in ("get", "post", "head", "options"):
        assert getattr(c, method)("/v1").status_code == 200


def test_content_parts_roles_and_backend_unavailable_and_rejection():
    c, fe = client(["ok"])
    body = dict(BODY, messages=[{"role": "developer", "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]},
                                {"role": "user", "content": "q"}])
    assert c.post("/v1/chat/completions", json=body).status_code == 200
    assert fe.submitted[0][0][0] == {"role": "system", "content": "ab"}
    assert c.post("/v1/chat/completions", json=dict(BODY, messages=[{"role": "tool", "content": "x"}])).status_code == 400
    fe.available = False
    r = c.post("/v1/chat/completions", json=BODY)
    assert r.status_code == 503 and r.json()["error"]["code"] == "backend_unavailable"
    c2, _ = client([""], "length_rejected")
    r = c2.post("/v1/chat/completions", json=BODY)
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"


def test_generate_route_streams_text_lines():
    c, _ = client(["a", "b"])
    with c.stream("POST", "/generate", json={"prompt": "p", "max_tokens": 4}) as r:
        lines = list(r.iter_lines())
    assert [l for l in lines if l] == ["data: a", "data: b", "data: [DONE]"]


def test_reasoning_parser_holds_back_partial_delimiter():
    p = ReasoningContentParser(True)
    assert p.feed("abc<") == ("abc", "")
    assert p.feed("/thi") == ("", "")
    assert p.feed("nk>z") == ("", "z")
    assert p.feed("more") == ("", "more")
    q = ReasoningContentParser(True)
    assert q.feed("x</") == ("x", "") and q.feed("b") == ("</b", "")
    assert ReasoningContentParser(False).feed("</think>") == ("", "</think>")


# ---------------------------------------------------------------------------- args
def test_args_aliases_recipes_and_shell_mode():
    a = parse_args(["--model-path", "/m/x", "--tp-size", "8", "--recipe", "high_m256", "--max-model-len", "4096",
                    "--graph", "64", "--max-extend-length", "4096", "--port", "2000"])
    assert a.model_path == "/m/x" and a.tp_info.size == 8 and a.recipe == "high_m256" and a.context_length == 4096
    assert a.cuda_graph_max_bs == 64 and a.max_extend_tokens == 4096 and a.max_running_req is UNSET
    assert a.model_names == ("x", "/m/x") and a.distributed_addr == "tcp://127.0.0.1:2001"
    assert "recipe" in a.explicit_fields and "max_running_req" not in a.explicit_fields
    s = parse_args(["--model", "/m/y", "--shell-mode"])
    assert s.shell_mode and s.max_running_req == 1 and s.cuda_graph_max_bs == 1
    assert parse_args(["--model", "/m/y", "--served-model-name", "zz"]).model_names == ("zz", "/m/y")
    assert parse_args(["--model", "/m/y", "--disable-pynccl"]).use_pynccl is False
    with pytest.raises(SystemExit):
        parse_args(["--model", "/m/y", "--recipe", "nope"])


def test_recipe_fills_only_unset_fields():
    from minisgl.engine.config import EngineConfig
    from minisgl.engine.engine import Engine

    c = Engine._adjust_config(EngineConfig(recipe="long_context_m8"))
    assert (c.max_running_req, c.cuda_graph_max_bs, c.context_length) == (8, 8, 1048576)
    c = Engine._adjust_config(EngineConfig(recipe="high_m256", max_running_req=32, context_length=1000))
    assert (c.max_running_req, c.cuda_graph_max_bs, c.context_length) == (32, 32, 1000)
    assert Engine._adjust_config(EngineConfig()).max_running_req == 128
    with pytest.raises(ValueError):
        Engine._adjust_config(EngineConfig(recipe="x"))


# ---------------------------------------------------------------------------- supervisor
def _child_ok(ack_queue=None, role="", **_):
    ack_queue.put(role)
    time.sleep(30)


def _child_exit_early(ack_queue=None, role="", **_):
    raise SystemExit(3)


def _child_hang(ack_queue=None, role="", **_):
    time.sleep(30)


def _child_ack_then_die(ack_queue=None, role="", **_):
    ack_queue.put(role)
    time.sleep(0.3)
    raise SystemExit(5)


def test_supervisor_ready_runtime_exit_and_idempotent_shutdown():
    sup = ServerProcessSupervisor(startup_timeout_s=20, mp_context="fork")
    sup.start([ProcessSpec("a", _child_ok), ProcessSpec("b", _child_ack_then_die)])
    assert sup.unexpected_exit() is None or sup.unexpected_exit()[0] == "b"
    time.sleep(0.8)
    assert sup.unexpected_exit() == ("b", 5)
    sup.shutdown()
    sup.shutdown()
    assert sup.alive_roles() == [] and sup.unexpected_exit() is None


def test_supervisor_startup_failures():
    sup = ServerProcessSupervisor(startup_timeout_s=20, mp_context="fork")
    with pytest.raises(SupervisorError, match="exited with code 3"):
        sup.start([ProcessSpec("a", _child_ok), ProcessSpec("bad", _child_exit_early)])
    assert sup.alive_roles() == []
    sup = ServerProcessSupervisor(startup_timeout_s=0.5, mp_context="fork")
    with pytest.raises(SupervisorError, match="not ready"):
        sup.start([ProcessSpec("h", _child_hang)])
    assert sup.alive_roles() == []
    with pytest.raises(SupervisorError, match="unique"):
        ServerProcessSupervisor(mp_context="fork").start([ProcessSpec("x", _child_ok), ProcessSpec("x", _child_ok)])


def test_frontend_marks_backend_unavailable_when_a_child_dies():
    from minisgl.server.api_server import FrontendManager

    class Sup:
        def __init__(self):
            self.dead, self.stopped = None, False

        def unexpected_exit(self):
            return self.dead

        def shutdown(self):
            self.stopped = True

    class Q:
        async def get(self):
            await asyncio.sleep(3600)

        async def put(self, m):
            pass

    async def run():
        sup = Sup()
        fm = FrontendManager(Q(), Q(), sup)
        fm.start()
        uid = await fm.submit("x", SamplingParams(), None)
        sup.dead = ("scheduler-0", -9)
        with pytest.raises(BackendUnavailable):
            async for _ in fm.stream(uid):
                pass
        assert not fm.available and sup.stopped
        with pytest.raises(BackendUnavailable):
            await fm.submit("y", SamplingParams(), None)
        await fm.stop()

    asyncio.run(run())


# ---------------------------------------------------------------------------- messages
def test_message_roundtrip():
    sp = SamplingParams(temperature=0.5, top_k=3, max_tokens=9)
    m = BatchBackendMsg([UserMsg(4, torch.arange(6, dtype=torch.int32), sp, "max"), AbortBackendMsg(2), ExitMsg()])
    r = unpack(pack(m))
    assert isinstance(r.data[0], UserMsg) and torch.equal(r.data[0].input_ids, torch.arange(6, dtype=torch.int32))
    assert r.data[0].sampling_params == sp and r.data[0].reasoning_effort == "max" and r.data[1].uid == 2
    t = unpack(pack(TokenizeMsg(1, [{"role": "user", "content": "x"}], sp, None)))
    assert t.text == [{"role": "user", "content": "x"}]
    d = unpack(pack(DetokenizeMsg(3, 17, True, "stop")))
    assert (d.uid, d.next_token, d.finished, d.finish_reason) == (3, 17, True, "stop")


def test_heartbeat_board_flags_a_wedged_rank_only_while_busy():
    """Liveness of running schedulers: a rank that reported work and then stops stamping is flagged; an idle rank and
    a rank that keeps stamping are not.  No GPU, no real hang: the clock is passed in."""
    from minisgl.utils.heartbeat import HeartbeatBoard

    board = HeartbeatBoard(None, 3, create=True)
    try:
        peer = HeartbeatBoard(board.name, 3, create=False)  # as a scheduler process attaches
        assert board.stale(10.0, now=1000.0) == []           # nobody has stamped yet
        peer.beat(0, busy=True, now=1000.0)
        peer.beat(1, busy=False, now=1000.0)                 # idle: blocked in receive
        peer.beat(2, busy=True, now=1000.0)
        assert board.stale(10.0, now=1005.0) == []
        peer.beat(2, busy=True, now=1050.0)                  # rank 2 keeps going, rank 0 went silent mid-work
        assert board.stale(10.0, now=1055.0) == [0]
        assert board.read(2)[0] == 2
        peer.shm.close()
    finally:
        board.close()


def test_frontend_marks_backend_unavailable_on_stale_heartbeat():
    import asyncio

    from minisgl.server.api_server import FrontendManager
    from minisgl.utils.heartbeat import HeartbeatBoard

    class Q:
        async def get(self):
            await asyncio.sleep(3600)

        async def put(self, m):
            pass

    board = HeartbeatBoard(None, 1, create=True)
    try:
        board.beat(0, busy=True, now=1.0)  # stamped long ago (epoch time 1 s), still "busy"

        async def run():
            f = FrontendManager(Q(), Q(), None)
            f.heartbeat, f.heartbeat_timeout = board, 5.0
            f.start()
            for _ in range(40):
                if not f.available:
                    break
                await asyncio.sleep(0.1)
            for t in f._tasks:
                t.cancel()
            return f

        f = asyncio.run(run())
        assert not f.available and "heartbeat" in f.unavailable_reason
    finally:
        board.close()
