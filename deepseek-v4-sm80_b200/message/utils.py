"""Dataclass <-> plain-dict serialisation for the ZMQ wire (msgpack carries the dicts).

Every message class registers itself; an encoded object is ``{"__type__": name, **fields}``; nested messages,
lists and dicts recurse; 1-D tensors travel as raw bytes with their dtype
(python/minisgl/message/utils.py:9-69 of the reference).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Type

import numpy as np
import torch

_REGISTRY: Dict[str, Type] = {}
_NP = {"int32": np.int32, "int64": np.int64, "float32": np.float32, "uint8": np.uint8}


def message(cls):
    cls = dataclasses.dataclass(cls)
    _REGISTRY[cls.__name__] = cls
    return cls


def encode(obj: Any) -> Any:
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        d = {"__type__": type(obj).__name__}
        for f in dataclasses.fields(obj):
            d[f.name] = encode(getattr(obj, f.name))
        return d
    if isinstance(obj, torch.Tensor):
        assert obj.dim() == 1, "only 1-D tensors are serialised"
        a = obj.detach().cpu().contiguous().numpy()
        return {"__type__": "__tensor__", "dtype": str(a.dtype), "data": a.tobytes()}
    if isinstance(obj, (list, tuple)):
        return [encode(x) for x in obj]
    if isinstance(obj, dict):
        return {k: encode(v) for k, v in obj.items()}
    return obj


def decode(obj: Any) -> Any:
    if isinstance(obj, dict):
        t = obj.get("__type__")
        if t == "__tensor__":
            return torch.from_numpy(np.frombuffer(obj["data"], dtype=_NP[obj["dtype"]]).copy())
        if t is not None:
            cls = _REGISTRY[t]
            return cls(**{k: decode(v) for k, v in obj.items() if k != "__type__"})
        return {k: decode(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [decode(x) for x in obj]
    return obj


def pack(obj: Any) -> bytes:
    import msgpack

    return msgpack.packb(encode(obj), use_bin_type=True)


def unpack(data: bytes) -> Any:
    import msgpack

    return decode(msgpack.unpackb(data, raw=False))
