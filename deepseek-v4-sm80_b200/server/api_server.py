"""OpenAI-compatible HTTP frontend.

Routes: ``POST /v1/chat/completions`` (streaming and non-streaming), ``GET /v1/models``, ``GET|POST|HEAD|OPTIONS /v1``,
``POST /generate``.  The request schema forbids unknown fields; unsupported OpenAI parameters are answered with
HTTP 400 ``{"error": {"message", "type": "invalid_request_error", "param", "code"}}``; an unknown model name with 404
``model_not_found``; a dead backend with 503 ``backend_unavailable``.  ``reasoning_content`` is split from the
answer at ``</think>`` with hold-back of a partially received delimiter.  A client disconnect aborts its request.
The contract is the reference's (python/minisgl/server/api_server.py:66-1057); the implementation is organised
around ``create_app(frontend, args)`` so that tests can drive it with an in-process fake frontend.
"""
from __future__ import annotations

import asyncio
import json
import math
import time
import uuid
from dataclasses import dataclass
from typing import Any, AsyncIterator, Callable, Dict, List, Literal, Optional, Union

from fastapi import FastAPI, Request
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, Response, StreamingResponse
from pydantic import BaseModel, ConfigDict, ValidationError

from ..core import SamplingParams
from ..message import AbortMsg, BatchFrontendMsg, TokenizeMsg, UserReply
from ..utils.logger import init_logger

logger = init_logger(__name__)
THINK_END = "</think>"


# --------------------------------------------------------------------------- schemas
class TextPart(BaseModel):
    model_config = ConfigDict(extra="forbid")
    type: Literal["text"]
    text: str


class ChatMessage(BaseModel):
    model_config = ConfigDict(extra="forbid")
    role: Literal["system", "developer", "user", "assistant"]
    content: Union[str, List[TextPart], None] = None
    reasoning_content: Optional[str] = None
    name: Optional[str] = None

    def to_plain(self) -> dict:
        c = self.content
        if isinstance(c, list):
            c = "".join(p.text for p in c)
        d = {"role": "system" if self.role == "developer" else self.role, "content": c or ""}
        if self.reasoning_content is not None:
            d["reasoning_content"] = self.reasoning_content
        return d


class StreamOptions(BaseModel):
    model_config = ConfigDict(extra="forbid")
    include_usage: bool = False


class OpenAICompletionRequest(BaseModel):
    model_config = ConfigDict(extra="forbid")
    model: str
    messages: Optional[List[ChatMessage]] = None
    prompt: Any = None
    max_tokens: Optional[int] = None
    max_completion_tokens: Optional[int] = None
    reasoning_effort: Optional[Literal["none", "high", "max"]] = None
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    n: int = 1
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    stop: Any = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    ignore_eos: bool = False
    user: Optional[str] = None
    metadata: Optional[Dict[str, Any]] = None
    # accepted by the schema only so that they can be refused with a precise message
    tools: Any = None
    tool_choice: Any = None
    parallel_tool_calls: Any = None
    functions: Any = None
    function_call: Any = None
    response_format: Any = None
    logprobs: Any = None
    top_logprobs: Any = None
    logit_bias: Any = None
    modalities: Any = None
    audio: Any = None
    prediction: Any = None
    seed: Any = None


class GenerateRequest(BaseModel):
    model_config = ConfigDict(extra="forbid")
    prompt: str
    max_tokens: int = 2048
    ignore_eos: bool = False


UNSUPPORTED = ("tools", "tool_choice", "parallel_tool_calls", "functions", "function_call", "response_format",
               "top_logprobs", "logit_bias", "modalities", "audio", "prediction", "seed")
DEFAULT_MAX_TOKENS = 2048


class APIError(Exception):
    def __init__(self, status: int, message: str, code: str, param: Optional[str] = None,
                 etype: str = "invalid_request_error"):
        self.status, self.message, self.code, self.param, self.etype = status, message, code, param, etype

    def response(self) -> JSONResponse:
        return JSONResponse(status_code=self.status, content={
            "error": {"message": self.message, "type": self.etype, "param": self.param, "code": self.code}})


def _bad(msg: str, param: Optional[str], code: str = "unsupported_parameter") -> APIError:
    return APIError(400, msg, code, param)


def validate_request(req: OpenAICompletionRequest) -> SamplingParams:
    """Semantic checks after schema validation; returns the sampling parameters."""
    if req.prompt is not None:
        raise _bad("'prompt' is not supported on /v1/chat/completions; send 'messages'", "prompt")
    for name in UNSUPPORTED:
        if getattr(req, name) is not None:
            raise _bad(f"'{name}' is not supported by this server", name)
    if req.logprobs:
        raise _bad("'logprobs' is not supported by this server", "logprobs")
    if not req.messages:
        raise _bad("'messages' must contain at least one message", "messages", "invalid_value")
    if req.n != 1:
        raise _bad("only n=1 is supported", "n", "invalid_value")
    if req.stop not in (None, [], ""):
        raise _bad("'stop' sequences are not supported", "stop")
    if req.presence_penalty != 0 or req.frequency_penalty != 0:
        which = "presence_penalty" if req.presence_penalty != 0 else "frequency_penalty"
        raise _bad(f"'{which}' must be 0", which, "invalid_value")
    if not math.isfinite(req.temperature) or req.temperature < 0:
        raise _bad("'temperature' must be a finite number >= 0", "temperature", "invalid_value")
    if not (req.top_k == -1 or req.top_k > 0):
        raise _bad("'top_k' must be -1 or a positive integer", "top_k", "invalid_value")
    if not 0.0 <= req.top_p <= 1.0:
        raise _bad("'top_p' must be in [0, 1]", "top_p", "invalid_value")
    max_tokens = req.max_completion_tokens if req.max_completion_tokens is not None else req.max_tokens
    if max_tokens is None:
        max_tokens = DEFAULT_MAX_TOKENS
    if max_tokens < 1:
        raise _bad("'max_tokens' must be at least 1", "max_tokens", "invalid_value")
    return SamplingParams(temperature=req.temperature, top_k=req.top_k, top_p=req.top_p, ignore_eos=req.ignore_eos,
                          max_tokens=max_tokens)


def param_from_validation_error(e: ValidationError) -> Optional[str]:
    errs = e.errors()
    if not errs:
        return None
    loc = [str(x) for x in errs[0].get("loc", ()) if not isinstance(x, int)]
    return loc[0] if loc else None


# --------------------------------------------------------------------------- reasoning split
class ReasoningContentParser:
    """Splits a token stream into (reasoning, answer) at the first ``</think>``.  While thinking, a suffix that could
    be the beginning of the delimiter is held back until it is disambiguated."""

    def __init__(self, thinking: bool):
        self.thinking, self.hold = thinking, ""

    def feed(self, text: str, final: bool = False):
        """Returns (reasoning_delta, content_delta)."""
        if not self.thinking:
            return "", text
        buf = self.hold + text
        i = buf.find(THINK_END)
        if i >= 0:
            self.thinking, self.hold = False, ""
            return buf[:i], buf[i + len(THINK_END):]
        keep = 0
        if not final:
            for k in range(min(len(THINK_END) - 1, len(buf)), 0, -1):
                if THINK_END.startswith(buf[-k:]):
                    keep = k
                    break
        self.hold = buf[len(buf) - keep:] if keep else ""
        return buf[: len(buf) - keep], ""


# --------------------------------------------------------------------------- frontend manager
class BackendUnavailable(Exception):
    pass


class FrontendManager:
    """Owns the sockets to the tokenizer workers, assigns request ids and fans replies out to per-request queues."""

    def __init__(self, recv_queue, send_queue, supervisor=None):
        self.recv, self.send, self.supervisor = recv_queue, send_queue, supervisor
        self.uid = 0
        self.queues: Dict[int, asyncio.Queue] = {}
        self.available = True
        self.unavailable_reason: Optional[str] = None
        self._tasks: List[asyncio.Task] = []

    def start(self) -> None:
        self._tasks = [asyncio.create_task(self._listen()), asyncio.create_task(self._watch_child_health())]

    async def _listen(self) -> None:
        try:
            while True:
                msg = await self.recv.get()
                for r in (msg.data if isinstance(msg, BatchFrontendMsg) else [msg]):
                    q = self.queues.get(r.uid)
                    if q is not None:
                        q.put_nowait(r)
        except asyncio.CancelledError:
            raise
        except Exception as e:
            self.mark_backend_unavailable(f"reply listener died: {e!r}")

    async def _watch_child_health(self) -> None:
        while self.available:
            await asyncio.sleep(1.0)
            if self.supervisor is not None:
                dead = self.supervisor.unexpected_exit()
                if dead is not None:
                    self.mark_backend_unavailable(f"backend process {dead[0]} exited with code {dead[1]}")
            board = getattr(self, "heartbeat", None)
            if board is not None and self.available:
                wedged = board.stale(self.heartbeat_timeout)
                if wedged:
                    self.mark_backend_unavailable(f"scheduler rank(s) {wedged} stopped making progress "
                                                  f"(no heartbeat for {self.heartbeat_timeout:.0f} s while busy)")

    def mark_backend_unavailable(self, reason: str) -> None:
        """Terminal state: wake every waiter, refuse new work, stop the children."""
        if not self.available:
            return
        self.available, self.unavailable_reason = False, reason
        logger.error("backend unavailable: %s", reason)
        for q in self.queues.values():
            q.put_nowait(None)
        if self.supervisor is not None:
            try:
                self.supervisor.shutdown()
            except Exception as e:  # pragma: no cover
                logger.error("forced shutdown failed: %s", e)

    async def submit(self, text: Any, sampling: SamplingParams, reasoning_effort: Optional[str]) -> int:
        if not self.available:
            raise BackendUnavailable(self.unavailable_reason or "backend unavailable")
        uid = self.uid
        self.uid += 1
        self.queues[uid] = asyncio.Queue()
        try:
            await self.send.put(TokenizeMsg(uid, text, sampling, reasoning_effort))
        except Exception as e:
            self.queues.pop(uid, None)
            self.mark_backend_unavailable(f"send to tokenizer failed: {e!r}")
            raise BackendUnavailable(self.unavailable_reason)
        return uid

    async def stream(self, uid: int) -> AsyncIterator[UserReply]:
        q = self.queues[uid]
        try:
            while True:
                r = await q.get()
                if r is None:
                    raise BackendUnavailable(self.unavailable_reason or "backend unavailable")
                yield r
                if r.finished:
                    return
        finally:
            self.queues.pop(uid, None)

    async def abort(self, uid: int) -> None:
        self.queues.pop(uid, None)
        if self.available:
            try:
                await self.send.put(AbortMsg(uid))
            except Exception:  # pragma: no cover
                pass

    async def stop(self) -> None:
        for t in self._tasks:
            t.cancel()


# --------------------------------------------------------------------------- app
@dataclass
class ServeInfo:
    model_names: tuple
    root: str


def _chunk(cid: str, model: str, created: int, delta: dict, finish: Optional[str] = None, usage=None,
           choices: bool = True) -> str:
    body = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model,
            "choices": [{"index": 0, "delta": delta, "finish_reason": finish}] if choices else []}
    if usage is not None:
        body["usage"] = usage
    return f"data: {json.dumps(body, ensure_ascii=False)}\n\n"


def create_app(frontend, info: ServeInfo) -> FastAPI:
    app = FastAPI(title="minisgl (B200)")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])

    @app.exception_handler(APIError)
    async def _api_error(_: Request, e: APIError):
        return e.response()

    @app.exception_handler(BackendUnavailable)
    async def _unavailable(_: Request, e: BackendUnavailable):
        return APIError(503, f"backend unavailable: {e}", "backend_unavailable", None, "server_error").response()

    @app.api_route("/v1", methods=["GET", "POST", "HEAD", "OPTIONS"])
    async def v1_root():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": info.model_names[0], "object": "model", "created": 0,
                                            "owned_by": "mini-sglang", "root": info.root}]}

    @app.post("/generate")
    async def generate(request: Request):
        try:
            req = GenerateRequest.model_validate(await request.json())
        except ValidationError as e:
            raise _bad(str(e.errors()[0].get("msg", "invalid request")), param_from_validation_error(e), "invalid_value")
        sp = SamplingParams(max_tokens=req.max_tokens, ignore_eos=req.ignore_eos)
        uid = await frontend.submit(req.prompt, sp, None)

        async def gen():
            try:
                async for r in frontend.stream(uid):
                    if await request.is_disconnected():
                        await frontend.abort(uid)
                        return
                    if r.incremental_output:
                        yield f"data: {r.incremental_output}\n"
                yield "data: [DONE]\n"
            except asyncio.CancelledError:
                await frontend.abort(uid)
                raise

        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/chat/completions")
    async def v1_completions(request: Request):
        try:
            payload = await request.json()
        except Exception:
            raise _bad("request body must be JSON", None, "invalid_json")
        try:
            req = OpenAICompletionRequest.model_validate(payload)
        except ValidationError as e:
            err = e.errors()[0]
            param = param_from_validation_error(e)
            code = "unknown_parameter" if err.get("type") == "extra_forbidden" else "invalid_value"
            raise APIError(400, f"{param}: {err.get('msg', 'invalid value')}" if param else str(err.get("msg")), code,
                           param)
        if req.model not in info.model_names:
            raise APIError(404, f"The model '{req.model}' does not exist", "model_not_found", "model")
        sp = validate_request(req)
        effort = None if req.reasoning_effort in (None, "none") else req.reasoning_effort
        messages = [m.to_plain() for m in req.messages]
        if not getattr(frontend, "available", True):
            raise BackendUnavailable(getattr(frontend, "unavailable_reason", None) or "backend unavailable")
        uid = await frontend.submit(messages, sp, effort)
        cid, created = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        model = req.model
        parser = ReasoningContentParser(thinking=effort is not None)

        def usage_of(n_out: int, n_in: int = 0) -> dict:
            return {"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out}

        if req.stream:
            async def sse():
                n_out, n_in, finish = 0, 0, None
                try:
                    yield _chunk(cid, model, created, {"role": "assistant", "content": ""})
                    async for r in frontend.stream(uid):
                        if await request.is_disconnected():
                            await frontend.abort(uid)
                            return
                        if r.finish_reason == "length_rejected":
                            yield f"data: {json.dumps({'error': {'message': 'prompt exceeds the context length', 'type': 'invalid_request_error', 'param': 'messages', 'code': 'context_length_exceeded'}})}\n\n"
                            yield "data: [DONE]\n\n"
                            return
                        n_out = r.num_tokens or n_out
                        n_in = r.prompt_tokens or n_in
                        rs, ct = parser.feed(r.incremental_output, final=r.finished)
                        if rs:
                            yield _chunk(cid, model, created, {"reasoning_content": rs})
                        if ct:
                            yield _chunk(cid, model, created, {"content": ct})
                        if r.finished:
                            finish = "length" if r.finish_reason == "length" else "stop"
                    yield _chunk(cid, model, created, {}, finish or "stop")
                    if req.stream_options and req.stream_options.include_usage:
                        yield _chunk(cid, model, created, {}, usage=usage_of(n_out, n_in), choices=False)
                    yield "data: [DONE]\n\n"
                except BackendUnavailable as e:
                    yield f"data: {json.dumps({'error': {'message': str(e), 'type': 'server_error', 'param': None, 'code': 'backend_unavailable'}})}\n\n"
                except asyncio.CancelledError:
                    await frontend.abort(uid)
                    raise

            return StreamingResponse(sse(), media_type="text/event-stream")

        reasoning, content, n_out, n_in, finish = [], [], 0, 0, "stop"
        try:
            async for r in frontend.stream(uid):
                if await request.is_disconnected():
                    await frontend.abort(uid)
                    return Response(status_code=499)
                if r.finish_reason == "length_rejected":
                    raise APIError(400, "prompt exceeds the model's maximum context length", "context_length_exceeded",
                                   "messages")
                if r.finished and r.finish_reason not in (None, "stop", "length", "abort"):
                    raise APIError(500, f"backend error: {r.finish_reason}", "backend_error", None, "server_error")
                n_out = r.num_tokens or n_out
                n_in = r.prompt_tokens or n_in
                rs, ct = parser.feed(r.incremental_output, final=r.finished)
                reasoning.append(rs)
                content.append(ct)
                if r.finished:
                    finish = "length" if r.finish_reason == "length" else "stop"
        except asyncio.CancelledError:
            await frontend.abort(uid)
            raise
        message = {"role": "assistant", "content": "".join(content)}
        if effort is not None:
            message["reasoning_content"] = "".join(reasoning)
        return {"id": cid, "object": "chat.completion", "created": created, "model": model,
                "choices": [{"index": 0, "message": message, "finish_reason": finish}], "usage": usage_of(n_out, n_in)}

    return app


# --------------------------------------------------------------------------- shell + runner
async def shell(frontend, args) -> None:
    """Minimal interactive chat loop (the reference uses prompt_toolkit; plain input() keeps this dependency-free)."""
    from ..env import ENV

    history: List[dict] = []
    loop = asyncio.get_running_loop()
    print("minisgl shell -- /reset clears the conversation, /exit quits")
    while True:
        try:
            line = (await loop.run_in_executor(None, input, "> ")).strip()
        except (EOFError, KeyboardInterrupt):
            break
        if line in ("/exit", "/quit"):
            break
        if line == "/reset":
            history.clear()
            continue
        if not line:
            continue
        history.append({"role": "user", "content": line})
        sp = SamplingParams(temperature=ENV.SHELL_TEMPERATURE.value, top_k=ENV.SHELL_TOP_K.value,
                            top_p=ENV.SHELL_TOP_P.value, max_tokens=ENV.SHELL_MAX_TOKENS.value)
        uid = await frontend.submit(list(history), sp, None)
        out = []
        async for r in frontend.stream(uid):
            print(r.incremental_output, end="", flush=True)
            out.append(r.incremental_output)
        print()
        history.append({"role": "assistant", "content": "".join(out)})


def run_api_server(args, start_backend: Callable[[], Any]) -> None:
    import uvicorn

    from ..utils.mp import ZmqAsyncPullQueue, ZmqAsyncPushQueue
    from .launch import graceful_exit_hook

    recv = ZmqAsyncPullQueue(args.zmq_frontend_addr, create=True)
    send_addr = args.zmq_detokenizer_addr if args.share_tokenizer else args.zmq_tokenizer_addr
    supervisor = start_backend()
    send = ZmqAsyncPushQueue(send_addr, create=False)
    frontend = FrontendManager(recv, send, supervisor)
    frontend.heartbeat = getattr(supervisor, "heartbeat", None)
    frontend.heartbeat_timeout = getattr(args, "heartbeat_timeout", 120.0)
    info = ServeInfo(args.model_names, args.model_path)
    app = create_app(frontend, info)

    @app.on_event("startup")
    async def _start():
        frontend.start()

    try:
        if args.shell_mode:
            async def main():
                frontend.start()
                await shell(frontend, args)

            asyncio.run(main())
        else:
            logger.info("serving %s on http://%s:%d", info.model_names[0], args.server_host, args.server_port)
            uvicorn.run(app, host=args.server_host, port=args.server_port, log_level="warning")
    finally:
        try:
            supervisor.shutdown(graceful=graceful_exit_hook(args))
        finally:
            recv.stop()
            send.stop()
