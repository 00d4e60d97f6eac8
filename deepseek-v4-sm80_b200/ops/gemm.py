"""Dense projection GEMMs: ``out[M,N] = x[M,K] @ w[N,K]^T``.

CUDA tensors run the hand-written tcgen05/TMEM kernels in ``csrc/gemm_tcgen05.cu``;
CPU tensors run the fp32 PyTorch statement of the same arithmetic, which is also the
oracle the GPU tests compare against.  These replace the reference's cuBLAS calls on
dequantised BF16 weight caches (python/minisgl/models/deepseek_v4.py:145-149).

Skinny problems (few output tiles, long K) are split along K so that the whole GPU streams the weight; the CTAs
of a tile form a thread-block cluster and add their partials in split order over distributed shared memory.
"""
from __future__ import annotations

import ctypes

import torch

from . import native as nv
from .native import I, L

_COUNTERS = {}
NUM_SMS_HINT = 148


def _as2d(x):
    return x.reshape(-1, x.shape[-1])


def _counters(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    c = _COUNTERS.get(key)
    if c is None:
        c = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        _COUNTERS[key] = c
    return c


def pick_tiling(m: int, n: int, k_tiles: int, batches: int, fp8: bool, bn: int = 0, splits: int = 0):
    """(tile width, K splits) that put roughly one CTA on every SM."""
    mt = max((m + 127) // 128 * batches, 1)      # m == 0 (nothing to do) must not divide by zero below
    if fp8 and mt == 1 and bn == 0 and splits == 0:
        return _pick_decode_fp8(n, k_tiles)
    if bn == 0:
        fill = NUM_SMS_HINT * 2 // 3
        if mt == 1:
            # One row tile (decode).  Every column tile re-reads the whole activation from L2, so wider tiles are
            # cheaper per byte; but a split costs a cluster launch and two cluster barriers (about 4 us measured, 8 us
            # for 8-way), so: no split when 32-wide tiles alone fill the GPU, else the widest tile that fills it with
            # at most 4 splits.
            # (FP8 follows the same rule since its block scales are applied by the MMA itself.)
            if (n + 31) // 32 >= fill:
                bn = 128 if (n + 127) // 128 >= fill else 64 if (n + 63) // 64 >= fill else 32
            else:
                smax = max(min(4, k_tiles // 4), 1)
                for cand in (128, 64, 32):
                    bn = cand
                    if ((n + cand - 1) // cand) * smax >= fill:
                        break
        elif mt * ((n + 127) // 128) >= fill:
            bn = 128  # the widest tile that still gives about one CTA per SM
        elif mt * ((n + 63) // 64) >= fill:
            bn = 64
        else:
            bn = 32
    if splits == 0:
        ctas = mt * ((n + bn - 1) // bn)
        splits = 1
        if ctas <= NUM_SMS_HINT // 2 and k_tiles >= 8:
            # the splits of a tile form one thread-block cluster (2, 4 or 8 CTAs) that reduces in shared memory
            want = max(min(NUM_SMS_HINT // ctas, k_tiles // 4, 4 if mt == 1 else 8), 1)
            splits = 8 if want >= 8 else 4 if want >= 4 else 2 if want >= 2 else 1
    if mt * ((n + bn - 1) // bn) > (1 << 16):
        splits = 1
    return bn, splits


# One row tile of FP8 activations (decode): what a k-tile costs is its bytes from L2 -- every CTA re-reads the 16 KiB
# activation tile next to its bn x 128 bytes of weights -- at the rate one CTA's TMA ring pulls (about 57 GB/s:
# 32 CTAs x 12 k-tiles x 32 KiB took 6.9 us, 32 x 32 x 32 KiB 18.2 us) or at the L2's aggregate rate when all SMs
# pull (about 5.3 TB/s: 164 MB in 31 us), whichever is slower; a K split adds the cluster launch and its two
# barriers (4 us up to four ways).  The widest tile moves the fewest bytes (a weight row costs 16384 / bn + 128
# bytes per k-tile) but needs K splits to put enough CTAs on the GPU.
_SM_GBS, _L2_GBS, _SPLIT_US = 57.0, 5300.0, {1: 0.0, 2: 4.0, 4: 4.0}


def _pick_decode_fp8(n: int, k_tiles: int):
    best = None
    for bn in (32, 64, 128):
        tiles = (n + bn - 1) // bn
        for splits in (1, 2, 4):
            if splits > 1 and (k_tiles // splits < 2 or tiles * splits > 2 * NUM_SMS_HINT):
                continue
            ctas = tiles * splits
            per_cta = -(-k_tiles // splits) * (16384 + bn * 128)
            waves = -(-ctas // NUM_SMS_HINT)
            t = max(waves * per_cta / (_SM_GBS * 1e3), ctas * per_cta / (_L2_GBS * 1e3)) + _SPLIT_US[splits]
            if best is None or t < best[0] - 1e-9:
                best = (t, bn, splits)
    return best[1], best[2]


def _ws(m, n, bn, batches, splits, device):
    """Workspace of the global-memory split-K reduction.  Splits of 2, 4 or 8 need none: they reduce inside a
    thread-block cluster.  Other split counts (only reachable by asking for them) use the workspace."""
    if splits <= 1 or splits in (2, 4, 8):
        return None, None
    elems = nv.cuda_lib().dsv4_gemm_splitk_ws_elems
    elems.restype = ctypes.c_longlong
    return (torch.empty(elems(I(m), I(n), I(bn), I(batches), I(splits)), dtype=torch.float32, device=device),
            _counters(device))


def gemm_bf16(x, w, out=None, out_dtype=torch.bfloat16, accumulate=False, bn=0, splits=0):
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
    bn, splits = pick_tiling(m, n, (k + 63) // 64, 1, False, bn, splits)
    ws, cnt = _ws(m, n, bn, 1, splits, x.device)
    nv.call("gemm_bf16", nv.ptr(x2), nv.ptr(w), nv.ptr(o2), I(m), I(n), I(k), I(x2.stride(0)), I(w.stride(0)),
            I(o2.stride(0)), I(1 if out.dtype == torch.float32 else 0), I(1 if accumulate else 0), I(bn), I(1),
            I(splits), nv.ptr(ws), nv.ptr(cnt))
    return out


def gemm_bf16_partials(x, w, splits: int = 0, gate=None):
    """Split-K bf16 GEMM that leaves the reduction to its consumer: returns fp32 [splits, M, N] with
    sum(0) == x @ w^T.  A split whose K range is empty writes zeros.  gate (a row-sharded exchange context): x is
    the gathered buffer and every CTA waits for its row block's all-gather flag before loading it."""
    x2 = _as2d(x)
    m, k = x2.shape
    n = w.shape[0]
    k_tiles = (k + 63) // 64
    if splits <= 0:
        ctas = max(((m + 127) // 128) * ((n + 31) // 32), 1)      # m may be 0 (a rank that owns no rows)
        splits = max(1, min(NUM_SMS_HINT // ctas, k_tiles // 4, 64))
    if not x.is_cuda:
        per = (k_tiles + splits - 1) // splits * 64
        xf, wf = x2.float(), w.float()
        return torch.stack([xf[:, s * per:(s + 1) * per] @ wf[:, s * per:(s + 1) * per].t() for s in range(splits)])
    assert x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x2.stride(-1) == 1 and w.stride(-1) == 1
    out = torch.empty(splits, m, n, dtype=torch.float32, device=x.device)
    if gate is not None:
        nv.call("gemm_bf16_partials_gated", nv.ptr(x2), nv.ptr(w), nv.ptr(out), I(m), I(n), I(k), I(x2.stride(0)),
                I(w.stride(0)), I(n), I(32), I(splits), L(m * n), ctypes.byref(gate))
        return out
    nv.call("gemm_bf16_partials", nv.ptr(x2), nv.ptr(w), nv.ptr(out), I(m), I(n), I(k), I(x2.stride(0)),
            I(w.stride(0)), I(n), I(32), I(splits), L(m * n))
    return out


def gemm_fp8_gated(xq, sx, wq, sw, gate):
    """``gemm_fp8`` whose activation operand is the gathered buffer of a row-sharded exchange: the all-gather is
    fused into the A-tile loads (each CTA waits for its row block's flag, weights stream meanwhile)."""
    m, k = xq.shape
    n = wq.shape[0]
    out = torch.empty(m, n, dtype=torch.bfloat16, device=xq.device)
    bn, _ = pick_tiling(m, n, k // 128, 1, True, 0, 1)
    nv.call("gemm_fp8_gated", nv.ptr(xq), nv.ptr(wq), nv.ptr(out), nv.ptr(sx), nv.ptr(sw), I(m), I(n), I(k),
            I(xq.stride(0)), I(wq.stride(0)), I(n), I(bn), ctypes.byref(gate))
    return out


def gemm_bf16_grouped(x, w, groups: int, out=None):
    """Per-group projection in one launch: x [T, G*K], w [G*N, K] -> out [T, G*N] with
    out[:, g*N:(g+1)*N] = x[:, g*K:(g+1)*K] @ w[g*N:(g+1)*N]^T  (the low-rank output projection wo_a; the reference
    runs it as torch.bmm, python/minisgl/models/deepseek_v4.py:235-263)."""
    t = x.shape[0]
    k = x.shape[1] // groups
    n = w.shape[0] // groups
    if not x.is_cuda:
        y = torch.einsum("tgk,gnk->tgn", x.reshape(t, groups, k).float(), w.reshape(groups, n, k).float())
        y = y.reshape(t, groups * n).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.is_contiguous() and w.is_contiguous() and x.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(t, groups * n, dtype=x.dtype, device=x.device)
    bn, splits = pick_tiling(t, n, (k + 63) // 64, groups, False, 0, 0)
    ws, cnt = _ws(t, n, bn, groups, splits, x.device)
    nv.call("gemm_bf16", nv.ptr(x), nv.ptr(w), nv.ptr(out), I(t), I(n), I(k), I(x.stride(0)), I(w.stride(0)),
            I(out.stride(0)), I(0), I(0), I(bn), I(groups), I(splits), nv.ptr(ws), nv.ptr(cnt))
    return out


def gemm_fp8(xq, sx, wq, sw, out=None, out_dtype=torch.bfloat16, accumulate=False, bn=0, splits=0):
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
    bn, splits = pick_tiling(m, n, k // 128, 1, True, bn, splits)
    ws, cnt = _ws(m, n, bn, 1, splits, xq.device)
    nv.call("gemm_fp8", nv.ptr(x2), nv.ptr(wq), nv.ptr(o2), nv.ptr(s2), nv.ptr(sw), I(m), I(n), I(k),
            I(x2.stride(0)), I(wq.stride(0)), I(o2.stride(0)), I(1 if out.dtype == torch.float32 else 0),
            I(1 if accumulate else 0), I(bn), I(splits), nv.ptr(ws), nv.ptr(cnt))
    return out
