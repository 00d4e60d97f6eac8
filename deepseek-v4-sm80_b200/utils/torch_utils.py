"""``torch_dtype`` default-dtype context and NVTX range decorator (python/minisgl/utils/torch_utils.py:11-37)."""
from __future__ import annotations

import contextlib
import functools
import os

import torch

NVTX_ENABLED = os.environ.get("MINISGL_NVTX", "0") == "1"


@contextlib.contextmanager
def torch_dtype(dtype: torch.dtype):
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(old)


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when MINISGL_NVTX=1 and CUDA is up; otherwise free."""
    on = NVTX_ENABLED and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def nvtx_annotate(name: str, layer_id_field: str | None = None):
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(self, *a, **k):
            label = name
            if layer_id_field is not None:
                label = f"{name}[{getattr(self, layer_id_field, '?')}]"
            with nvtx_range(label):
                return fn(self, *a, **k)

        return wrapped

    return deco
