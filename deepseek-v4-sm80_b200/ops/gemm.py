"""Dense projection GEMMs: ``out[M,N] = x[M,K] @ w[N,K]^T``.

CUDA tensors run the hand-written tcgen05/TMEM kernels in ``csrc/gemm_tcgen05.cu``;
CPU tensors run the fp32 PyTorch statement of the same arithmetic, which is also the
oracle the GPU tests compare against.  These replace the reference's cuBLAS calls on
dequantised BF16 weight caches (python/minisgl/models/deepseek_v4.py:145-149).
"""
from __future__ import annotations

import torch

from . import native as nv
from .native import I


def _as2d(x):
    return x.reshape(-1, x.shape[-1])


def gemm_bf16(x, w, out=None, out_dtype=torch.bfloat16, accumulate=False, bn=0):
    """bf16 x bf16 -> bf16 / fp32 with fp32 accumulation."""
    x2 = _as2d(x)
    m, k = x2.shape
    n = w.shape[0]
    if not x.is_cuda:
        y = (x2.float() @ w.float().t())
        if out is not None:
            y = y.reshape(out.shape)
            y = y + out.float() if accumulate else y
            out.copy_(y.to(out.dtype))
            return out
        return y.to(out_dtype).reshape(*x.shape[:-1], n)
    assert x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, (x2.dtype, w.dtype)
    assert x2.stride(-1) == 1 and w.stride(-1) == 1
    if out is None:
        out = torch.empty(*x.shape[:-1], n, dtype=out_dtype, device=x.device)
    o2 = out.reshape(-1, n) if out.is_contiguous() else out
    assert o2.stride(-1) == 1
    nv.call("gemm_bf16", nv.ptr(x2), nv.ptr(w), nv.ptr(o2), I(m), I(n), I(k), I(x2.stride(0)), I(w.stride(0)),
            I(o2.stride(0)), I(1 if out.dtype == torch.float32 else 0), I(1 if accumulate else 0), I(bn))
    return out


def gemm_fp8(xq, sx, wq, sw, out=None, out_dtype=torch.bfloat16, accumulate=False, bn=0):
    """e4m3 x e4m3 with block scales: xq [M,K] + sx fp32 [M,K/128]; wq [N,K] + sw fp32 [ceil(N/128), K/128]."""
    x2 = _as2d(xq)
    m, k = x2.shape
    n = wq.shape[0]
    s2 = sx.reshape(m, -1)
    if not xq.is_cuda:
        xf = x2.float().reshape(m, k // 128, 128) * s2.unsqueeze(-1)
        wf = wq.float() * sw.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
        y = xf.reshape(m, k) @ wf.t()
        return y.to(out_dtype).reshape(*xq.shape[:-1], n)
    assert s2.dtype == torch.float32 and sw.dtype == torch.float32 and s2.is_contiguous() and sw.is_contiguous()
    if out is None:
        out = torch.empty(*xq.shape[:-1], n, dtype=out_dtype, device=xq.device)
    o2 = out.reshape(-1, n)
    nv.call("gemm_fp8", nv.ptr(x2), nv.ptr(wq), nv.ptr(o2), nv.ptr(s2), nv.ptr(sw), I(m), I(n), I(k),
            I(x2.stride(0)), I(wq.stride(0)), I(o2.stride(0)), I(1 if out.dtype == torch.float32 else 0),
            I(1 if accumulate else 0), I(bn))
    return out
