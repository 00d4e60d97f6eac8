"""ZMQ message queues between the API server, the tokenizer workers and the schedulers.

One small class per direction; all of them speak msgpack over ipc sockets and use the message serde of
:mod:`minisgl.message.utils`.  ``stop`` closes with a short linger so that shutdown never blocks on a dead peer.
Same roles as python/minisgl/utils/mp.py:12-151 of the reference (Push/Pull between processes, Pub/Sub from
scheduler rank 0 to the other ranks).
"""
from __future__ import annotations

from typing import Any, Generic, Optional, TypeVar

import zmq
import zmq.asyncio

from ..message.utils import pack, unpack

T = TypeVar("T")


class _Endpoint(Generic[T]):
    KIND = zmq.PUSH
    ASYNC = False

    def __init__(self, addr: str, create: bool, send_timeout_ms: Optional[int] = None):
        self.addr, self.created = addr, create
        self.context = zmq.asyncio.Context() if self.ASYNC else zmq.Context()
        self.socket = self.context.socket(self.KIND)
        self.socket.setsockopt(zmq.LINGER, 1000)
        if send_timeout_ms is not None:
            self.socket.setsockopt(zmq.SNDTIMEO, send_timeout_ms)
        if self.KIND == zmq.SUB:
            self.socket.setsockopt_string(zmq.SUBSCRIBE, "")
        (self.socket.bind if create else self.socket.connect)(addr)

    def stop(self) -> None:
        try:
            self.socket.close()
            self.context.term()
        except Exception:  # pragma: no cover - best effort on shutdown
            pass
        if self.created and self.addr.startswith("ipc://"):  # the binder owns the socket file
            import os

            try:
                os.unlink(self.addr[len("ipc://"):])
            except OSError:
                pass


class ZmqPushQueue(_Endpoint[T]):
    KIND = zmq.PUSH

    def put(self, obj: T) -> None:
        self.socket.send(pack(obj), copy=False)

    def put_raw(self, raw: bytes) -> None:
        self.socket.send(raw, copy=False)


class ZmqPullQueue(_Endpoint[T]):
    KIND = zmq.PULL

    def get(self) -> T:
        return unpack(self.socket.recv())

    def get_raw(self) -> bytes:
        return self.socket.recv()

    @staticmethod
    def decode(raw: bytes) -> Any:
        return unpack(raw)

    def empty(self) -> bool:
        return self.socket.poll(timeout=0) == 0

    def poll(self, timeout_ms: int) -> bool:
        return self.socket.poll(timeout=timeout_ms) != 0


class ZmqPubQueue(ZmqPushQueue[T]):
    KIND = zmq.PUB


class ZmqSubQueue(ZmqPullQueue[T]):
    KIND = zmq.SUB


class ZmqAsyncPushQueue(_Endpoint[T]):
    KIND = zmq.PUSH
    ASYNC = True

    async def put(self, obj: T) -> None:
        await self.socket.send(pack(obj), copy=False)


class ZmqAsyncPullQueue(_Endpoint[T]):
    KIND = zmq.PULL
    ASYNC = True

    async def get(self) -> T:
        return unpack(await self.socket.recv())
