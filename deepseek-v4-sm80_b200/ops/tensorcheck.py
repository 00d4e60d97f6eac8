"""Declarative tensor checks at the boundary to the native kernels.

The launchers in ``csrc`` take raw pointers; a tensor of the wrong dtype, rank, stride or device would be read as
garbage, not rejected.  The wrappers in :mod:`minisgl.ops.cuda` therefore declare what every tensor argument must look
like and :func:`tensors` verifies the declaration before the launch:

    @tensors(q="bf16[T,H,512]", sink="f32[H]", topk_idx="?i32[T,K]")
    def attention(q, ..., sink, ..., topk_idx): ...

A spec is ``dtype[dim, ...]`` followed by an optional layout letter: ``c`` (default) contiguous, ``s`` only the last
dimension must have stride 1 (row-strided views), ``*`` any layout.  A dimension is a number (must match), a name
(bound on first use, must agree across all arguments of the call, like ``T`` above) or ``_`` (anything).  A leading
``?`` allows ``None``.  Several dtypes may be given as ``bf16|f32``.  All tensors of one call must live on the same
CUDA device.  The reference does the same at its C++ boundary with a symbolic TensorMatcher
(python/minisgl/kernel/csrc/include/minisgl/tensor.h:140-300); here the check sits in front of the ctypes call.
"""
from __future__ import annotations

import functools
import inspect
import re
from typing import Dict

import torch

DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i32": torch.int32,
          "i64": torch.int64, "u8": torch.uint8, "i8": torch.int8, "e4m3": torch.float8_e4m3fn}
_SPEC = re.compile(r"^(\?)?([a-z0-9|]+)\[([^\]]*)\]([cs*])?$")


class TensorSpecError(TypeError):
    pass


@functools.lru_cache(maxsize=None)
def _parse(spec: str):
    m = _SPEC.match(spec.replace(" ", ""))
    if m is None:
        raise ValueError(f"bad tensor spec {spec!r}")
    optional, dts, dims, layout = m.groups()
    dtypes = tuple(DTYPES[d] for d in dts.split("|"))
    dims = tuple(int(d) if d.isdigit() else d for d in dims.split(",")) if dims else ()
    return bool(optional), dtypes, dims, layout or "c"


def match(name: str, spec: str, t, bound: Dict[str, int], device=None):
    """Checks one tensor against its spec; binds / compares symbolic dimensions in ``bound``.  Returns the device."""
    optional, dtypes, dims, layout = _parse(spec)
    if t is None:
        if optional:
            return device
        raise TensorSpecError(f"{name}: a tensor is required ({spec})")
    if not isinstance(t, torch.Tensor):
        raise TensorSpecError(f"{name}: expected a tensor ({spec}), got {type(t).__name__}")
    if t.dtype not in dtypes:
        raise TensorSpecError(f"{name}: dtype {t.dtype} does not match {spec}")
    if t.dim() != len(dims):
        raise TensorSpecError(f"{name}: shape {tuple(t.shape)} does not have the rank of {spec}")
    for i, d in enumerate(dims):
        n = t.shape[i]
        if isinstance(d, int):
            if n != d:
                raise TensorSpecError(f"{name}: dimension {i} is {n}, {spec} wants {d}")
        elif d != "_":
            if bound.setdefault(d, n) != n:
                raise TensorSpecError(f"{name}: dimension {d} is {n} here but {bound[d]} in an earlier argument")
    if layout == "c" and not t.is_contiguous():
        raise TensorSpecError(f"{name}: must be contiguous ({spec}), strides {t.stride()}")
    if layout == "s" and t.dim() and t.numel() and t.stride(-1) != 1:
        raise TensorSpecError(f"{name}: the last dimension must have stride 1 ({spec}), strides {t.stride()}")
    if device is not None and t.device != device:
        raise TensorSpecError(f"{name}: on {t.device}, other arguments on {device}")
    return t.device


def tensors(**specs: str):
    """Decorator: verifies the named tensor arguments of every call against their specs."""
    for s in specs.values():
        _parse(s)

    def deco(fn):
        sig = inspect.signature(fn)
        missing = [k for k in specs if k not in sig.parameters]
        if missing:
            raise ValueError(f"{fn.__name__}: no parameter(s) {missing}")

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            ba = sig.bind(*args, **kwargs)
            ba.apply_defaults()
            bound: Dict[str, int] = {}
            device = None
            for name, spec in specs.items():
                device = match(f"{fn.__name__}({name})", spec, ba.arguments[name], bound, device)
            return fn(*args, **kwargs)

        wrapper.tensor_specs = dict(specs)
        return wrapper

    return deco
