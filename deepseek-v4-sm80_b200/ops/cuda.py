"""Python wrappers around the sm_100a kernels (one function per facade op in :mod:`minisgl.ops.api`).

Every function allocates its outputs with torch (caching allocator, so CUDA-graph capture sees static
addresses on replay) and launches on the current stream.  Nothing here falls back to PyTorch math.
"""
from __future__ import annotations

import ctypes
import math
import os as _os

import torch

from . import native as nv
from .native import F, I, L
from .ref import RopeSpec
from .tensorcheck import tensors


class RopeParams(ctypes.Structure):
    _fields_ = [("rotary_dim", ctypes.c_int), ("log_base", ctypes.c_float), ("use_scaling", ctypes.c_int),
                ("factor", ctypes.c_float), ("low", ctypes.c_float), ("scale_denom", ctypes.c_float)]


_ROPE_CACHE = {}


def rope_params(spec: RopeSpec) -> RopeParams:
    rp = _ROPE_CACHE.get(spec)
    if rp is None:
        rp = RopeParams(spec.rotary_dim, math.log(spec.base), 1 if spec.use_scaling else 0, spec.factor,
                        float(spec.low), spec.scale_denom)
        _ROPE_CACHE[spec] = rp
    return rp


_SMS = {}


def num_sms(device) -> int:
    i = torch.device(device).index or 0
    if i not in _SMS:
        _SMS[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SMS[i]


def _i32(t):
    assert t.dtype == torch.int32, t.dtype
    return nv.ptr(t)


# --------------------------------------------------------------------------- elementwise
def check_index(idx, lo: int, hi: int, tag: int) -> None:
    """Audit int32 indices against [lo, hi) on the device; a violation lands in the status word (code 2, tag, position)
    and is raised by the next ``native.assert_device_ok()``."""
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    nv.call("check_index", nv.ptr(idx), ctypes.c_longlong(idx.numel()), I(lo), I(hi), I(tag))


@tensors(ids="i32[T]", weight="bf16[_,H]", feedback="?i32[_]", slots="?i32[T]")
def embed(ids, weight, m: int, feedback=None, slots=None):
    """feedback / slots: row t embeds token feedback[slots[t]] and writes it to ids[t]."""
    t, h = ids.shape[0], weight.shape[1]
    out = torch.empty(t, m, h, dtype=weight.dtype, device=weight.device)
    nv.call("embed", _i32(ids), nv.ptr(feedback), nv.ptr(slots), nv.ptr(weight), nv.ptr(out), I(t), I(m), I(h))
    return out


@tensors(logits="f32[R,_]s", slots="i32[R]", num_valid="?i32[1]", token_feedback="i32[_]", out="?i32[R]")
def greedy_tokens(logits, v_base: int, slots, num_valid, token_feedback, out=None, comm_ctx=None):
    """Argmax of fp32 logits rows (this rank's vocabulary shard starting at token v_base; with comm_ctx the shards'
    candidates are exchanged inside the kernel), written to out [rows] int32 and to token_feedback[slots[row]]."""
    rows, v = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    nv.call("greedy_tokens", nv.ptr(logits), I(logits.stride(0)), I(v), I(v_base), _i32(slots), nv.ptr(num_valid),
            _i32(token_feedback), _i32(out), I(rows), ctypes.byref(comm_ctx) if comm_ctx is not None else None)
    return out


def _quant_out(rows, d, device, want_q):
    if not want_q or d % 256:
        return None, None
    return (torch.empty(rows, d, dtype=torch.float8_e4m3fn, device=device),
            torch.empty(rows, d // 128, dtype=torch.float32, device=device))


def rms_norm(x, weight, eps: float, want_q: bool = False):
    """want_q: also returns the (e4m3, scales) quantisation of the result, written by the same kernel."""
    d = x.shape[-1]
    x2 = x if x.dim() == 2 else x.reshape(-1, d)
    assert x2.stride(-1) == 1
    out = torch.empty(x2.shape[0], d, dtype=x.dtype, device=x.device)
    q, s = _quant_out(x2.shape[0], d, x.device, want_q)
    nv.call("rms_norm", nv.ptr(x2), I(x2.stride(0)), nv.ptr(weight), nv.ptr(out), I(d), I(x2.shape[0]), I(d), F(eps),
            nv.ptr(q), nv.ptr(s))
    out = out.reshape(*x.shape[:-1], d)
    if want_q:
        return out, ((q, s) if q is not None else fp8_quant(out))
    return out


def fp8_quant(x, block: int = 128):
    k = x.shape[-1]
    x2 = x if x.dim() == 2 else x.reshape(-1, k)
    assert x2.stride(-1) == 1
    rows = x2.shape[0]
    q = torch.empty(rows, k, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(rows, k // block, dtype=torch.float32, device=x.device)
    nv.call("fp8_quant", nv.ptr(x2), I(x2.stride(0)), nv.ptr(q), nv.ptr(s), I(rows), I(k), I(block))
    return q, s


@tensors(gate_up="bf16[_,_]")
def silu_mul_clamp(gate_up, limit):
    rows, two_i = gate_up.shape
    out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    nv.call("silu_mul_clamp", nv.ptr(gate_up), nv.ptr(out), I(rows), I(two_i // 2), F(limit or 0.0))
    return out


@tensors(gate_up="bf16[_,_]")
def silu_mul_clamp_quant(gate_up, limit):
    """SwiGLU with clamp straight to (e4m3, scales); the bf16 activation is not materialised."""
    rows, two_i = gate_up.shape
    inter = two_i // 2
    if inter % 128:
        return fp8_quant(silu_mul_clamp(gate_up, limit))
    q = torch.empty(rows, inter, dtype=torch.float8_e4m3fn, device=gate_up.device)
    s = torch.empty(rows, inter // 128, dtype=torch.float32, device=gate_up.device)
    nv.call("silu_mul_clamp_quant", nv.ptr(gate_up), nv.ptr(q), nv.ptr(s), I(rows), I(inter), F(limit or 0.0))
    return q, s


@tensors(routed="bf16[R,H]", shared="bf16[R,H]", num_valid="?i32[1]")
def add_cast(routed, shared, num_valid=None):
    out = torch.empty_like(routed)
    nv.call("add_cast", nv.ptr(routed), nv.ptr(shared), nv.ptr(out), I(routed.shape[0]), I(routed.shape[1]),
            nv.ptr(num_valid))
    return out


def rope_tail(x, positions, spec, inverse: bool = False, pos_offset: int = 0):
    assert x.is_contiguous()
    d = x.shape[-1]
    rows = x.numel() // d
    heads = rows // positions.shape[0]
    nv.call("rope_tail", nv.ptr(x), _i32(positions), I(rows), I(heads), I(d), rope_params(spec),
            I(1 if inverse else 0), I(pos_offset))
    return x


@tensors(q="bf16[T,_,D]", kv="bf16[T,D]s", positions="i32[T]", kv_w="bf16[D]", swa_cache="bf16[_,D]", out_loc="i32[T]",
         swa_map="i32[_]")
def q_kv_norm_rope_store(q, kv, positions, kv_w, eps, spec, swa_cache, out_loc, swa_map, ps: int, qat: bool):
    t, h, d = q.shape
    assert q.is_contiguous() and kv.stride(-1) == 1
    nv.call("q_kv_norm_rope_store", nv.ptr(q), nv.ptr(kv), I(kv.stride(0)), _i32(positions), nv.ptr(kv_w), F(eps),
            rope_params(spec), nv.ptr(swa_cache), _i32(out_loc), _i32(swa_map), I(ps), I(t), I(h), I(d),
            I(1 if qat else 0))
    return q, kv


# --------------------------------------------------------------------------- hyper-connections
def _hc_mixes(x, fn):
    """Split-K partial products [S, t, MIX] of flatten(x[t]) . fn^T: one tensor-core GEMM over all tokens, whose
    splits the per-token kernel adds up."""
    from .gemm import gemm_bf16_partials

    t = x.shape[0]
    return gemm_bf16_partials(x.reshape(t, -1), fn)


@tensors(x="bf16[T,4,H]", fn="bf16[_,_]", scale="f32[_]", base="f32[_]", norm_w="?bf16[H]")
def hc_pre(x, fn, scale, base, iters, eps, norm_eps, norm_w=None, want_q: bool = False, out=None):
    """out = (y, q, s): preallocated result rows (the row-sharded layer passes its rows of the gathered buffer)."""
    t, m, h = x.shape
    assert m == 4 and x.is_contiguous()
    if out is not None:
        y, q, s = out
        assert y.shape == (t, h) and y.is_contiguous() and q.is_contiguous() and s.is_contiguous() and h % 256 == 0
    else:
        y = torch.empty(t, h, dtype=x.dtype, device=x.device)
        q, s = _quant_out(t, h, x.device, want_q)
    post = torch.empty(t, m, dtype=torch.float32, device=x.device)
    comb = torch.empty(t, m, m, dtype=torch.float32, device=x.device)
    mixes = _hc_mixes(x, fn)
    nv.call("hc_pre", nv.ptr(x), nv.ptr(fn), nv.ptr(mixes), I(mixes.stride(1)), I(mixes.shape[0]),
            L(mixes.stride(0)), nv.ptr(scale), nv.ptr(base),
            nv.ptr(norm_w), nv.ptr(y), nv.ptr(post), nv.ptr(comb), I(t), I(h), I(24), I(iters), F(eps), F(norm_eps),
            F(norm_eps), nv.ptr(q), nv.ptr(s))
    if want_q:
        return y, post, comb, ((q, s) if q is not None else fp8_quant(y))
    return y, post, comb


@tensors(y="bf16[T,H]", residual="bf16[T,4,H]", post="f32[T,4]", comb="f32[T,4,4]")
def hc_post(y, residual, post, comb):
    t, m, h = residual.shape
    out = torch.empty_like(residual)
    nv.call("hc_post", nv.ptr(y), nv.ptr(residual), nv.ptr(post), nv.ptr(comb), nv.ptr(out), I(t), I(h))
    return out


def hc_head(x, fn, scale, base, eps, norm_eps, norm_w=None):
    t, m, h = x.shape
    x = x.contiguous()
    y = torch.empty(t, h, dtype=x.dtype, device=x.device)
    mixes = _hc_mixes(x, fn)
    nv.call("hc_pre", nv.ptr(x), nv.ptr(fn), nv.ptr(mixes), I(mixes.stride(1)), I(mixes.shape[0]),
            L(mixes.stride(0)), nv.ptr(scale), nv.ptr(base),
            nv.ptr(norm_w), nv.ptr(y), nv.ptr(None), nv.ptr(None), I(t), I(h), I(4), I(0), F(eps), F(norm_eps),
            F(norm_eps), nv.ptr(None), nv.ptr(None))
    return y


# --------------------------------------------------------------------------- compressors / indexer producers
def compress(proj, fb, ratio: int, d: int, ape, ring, ckpt, ps: int):
    t = proj.shape[0]
    assert proj.stride(1) == 1 and proj.dtype == torch.float32  # may be a column slice of a wider GEMM output
    out = torch.empty(t, d, dtype=torch.float32, device=proj.device)
    pt = fb.page_table
    nv.call("compress_pool", nv.ptr(proj), I(proj.stride(0)), _i32(fb.positions), _i32(fb.slots), _i32(pt), I(pt.stride(0)),
            nv.ptr(ring), nv.ptr(ckpt), nv.ptr(ape), nv.ptr(out), I(t), I(d), I(ratio), I(ps))
    nv.call("compress_state", nv.ptr(proj), I(proj.stride(0)), _i32(fb.positions), _i32(fb.slots), _i32(pt), I(pt.stride(0)),
            nv.ptr(ring), nv.ptr(ckpt), nv.ptr(ape), I(t), I(d), I(ratio), I(ps))
    return out


def compress_store(pooled, fb, norm_w, eps, spec, cache, ps: int, ratio: int):
    t, d = pooled.shape
    nv.call("compress_store", nv.ptr(pooled), _i32(fb.positions), _i32(fb.out_loc), nv.ptr(norm_w), F(eps),
            rope_params(spec), nv.ptr(cache), I(t), I(d), I(ps), I(ratio))


@tensors(q="bf16[T,HI,DI]", weights="bf16[T,HI]", positions="i32[T]")
def indexer_q_encode(q, weights, positions, spec, softmax_scale, head_scale):
    t, h, d = q.shape
    assert q.is_contiguous() and weights.is_contiguous() and weights.dtype == torch.bfloat16
    codes = torch.empty(t, h, d, dtype=torch.uint8, device=q.device)
    wf = torch.empty(t, h, dtype=torch.float32, device=q.device)
    nv.call("indexer_q_encode", nv.ptr(q), nv.ptr(weights), _i32(positions), rope_params(spec),
            F(softmax_scale * head_scale), nv.ptr(codes), nv.ptr(wf), I(t), I(h), I(d))
    return codes, wf


def indexer_kv_store(pooled, fb, norm_w, eps, spec, vals, scales, ps: int):
    t, d = pooled.shape
    nv.call("indexer_kv_store", nv.ptr(pooled), _i32(fb.positions), _i32(fb.out_loc), nv.ptr(norm_w), F(eps),
            rope_params(spec), nv.ptr(vals), nv.ptr(scales), I(t), I(d), I(ps))


LOGITS_WORKSPACE_BYTES = 512 << 20   # bound of the fp32 logits workspace of one indexer call (rows are chunked)


def _mma_indexer_ok(h: int, d: int, ps: int) -> bool:
    rpp = ps // 4
    return h == 64 and d == 128 and ps % 4 == 0 and rpp >= 8 and (64 % rpp == 0 or rpp % 64 == 0)


@tensors(qc="u8[T,HI,DI]", wf="f32[T,HI]", vals="u8[_,DI]", scales="f32[_]", slots="i32[T]", positions="i32[T]",
         pt="i32[_,_]s", out="?f32[T,_]s")
def indexer_logits(qc, wf, vals, scales, slots, positions, pt, ps: int, width: int, prefill: bool, out=None,
                   force_scalar: bool = False):
    """fp32 logits [t, width] of the rows' compressed history (-inf past each row's length).  64 x 128 indexers run
    on the tensor cores (csrc/indexer_mma.cu); other shapes on the CUDA-core kernel."""
    t, h, d = qc.shape
    logits = out if out is not None else torch.empty(t, width, dtype=torch.float32, device=qc.device)
    if _mma_indexer_ok(h, d, ps) and not force_scalar:
        tg = 4 if (prefill and t >= 4) else 1
        groups = (t + tg - 1) // tg
        nblocks = (width + 127) // 128
        # one-token groups fit three CTAs on an SM (smaller ring, 128 tensor-memory columns), wider groups one
        ctas = (3 if tg == 1 else 2) * num_sms(qc.device)
        nsplit = max(1, min(nblocks, -(-ctas // groups)))
        nv.call("indexer_logits_mma", nv.ptr(qc), nv.ptr(wf), nv.ptr(vals), nv.ptr(scales), L(vals.shape[0]),
                _i32(slots), _i32(positions), _i32(pt), I(pt.stride(0)), I(ps), nv.ptr(logits), I(width), I(t), I(h),
                I(d), I(tg), I(nsplit))
    else:
        nv.call("indexer_logits", nv.ptr(qc), nv.ptr(wf), nv.ptr(vals), nv.ptr(scales), _i32(slots), _i32(positions),
                _i32(pt), I(pt.stride(0)), I(ps), nv.ptr(logits), I(width), I(t), I(h), I(d))
    return logits


def indexer_select(qc, wf, vals, scales, fb, ps: int, k: int):
    t, h, d = qc.shape
    idx = torch.empty(t, k, dtype=torch.int32, device=qc.device)
    out_len = torch.empty(t, dtype=torch.int32, device=qc.device)
    n_max = fb.max_context // 4
    if n_max <= k:
        # every row keeps its whole history: the selection is the identity and no logits are needed
        nv.call("topk", nv.ptr(None), I(k), _i32(fb.positions), nv.ptr(idx), nv.ptr(out_len), I(t), I(k))
        return idx, out_len
    width = (n_max + 63) // 64 * 64
    # The workspace is t x width floats; at a million tokens of context a row is 1 MiB, so the rows are processed in
    # chunks that keep it within LOGITS_WORKSPACE_BYTES (the reference bounds its workspace the same way,
    # python/minisgl/kernel/deepseek_v4.py:883-927).
    rows = max(1, min(t, LOGITS_WORKSPACE_BYTES // (width * 4)))
    if 4 <= rows < t:
        rows -= rows % 4        # whole groups of four rows per chunk
    pt = fb.page_table
    logits = torch.empty(rows, width, dtype=torch.float32, device=qc.device)
    for a in range(0, t, rows):
        b = min(a + rows, t)
        n = b - a
        indexer_logits(qc[a:b], wf[a:b], vals, scales, fb.slots[a:b], fb.positions[a:b], pt, ps, width,
                       bool(getattr(fb, "is_prefill", False)), out=logits[:n])
        nv.call("topk", nv.ptr(logits), I(width), _i32(fb.positions[a:b]), nv.ptr(idx[a:b]), nv.ptr(out_len[a:b]),
                I(n), I(k))
    return idx, out_len


# --------------------------------------------------------------------------- attention
_ATTN_COUNTERS = {}


def attention_splits(t: int, heads: int, mode: int, ratio: int, topk_width: int, window: int, max_context: int,
                     prefill: bool, sms: int) -> int:
    """CTAs per token.  Splitting pays when the tokens alone leave SMs idle and a token has many key tiles (decode of
    a few long sequences); a batch that fills the GPU, and every prefill chunk, runs one CTA per token."""
    if prefill or t <= 0:
        return 1
    keys = window + (topk_width if mode == 1 else (max_context // ratio if mode == 2 else 0))
    kt = 64 if heads <= 16 else 32          # keys per tile of the kernel's configuration
    ntiles = -(-keys // kt)
    return int(max(1, min(sms // t, -(-ntiles // 2), 32)))


@tensors(q="bf16[T,H,512]", swa_cache="bf16[_,512]", swa_map="i32[_]", comp_cache="?bf16[_,512]", topk_idx="?i32[T,_]",
         topk_len="?i32[T]", sink="f32[H]")
def attention(q, fb, swa_cache, swa_map, comp_cache, ratio: int, topk_idx, topk_len, sink, scale, ps: int,
              window: int, out_rope=None, nsplit: int = 0):
    """out_rope: RopeSpec whose inverse rotation the kernel applies to the tail of every output row.
    nsplit: CTAs per token (0: chosen by :func:`attention_splits`)."""
    t, h, d = q.shape
    o = torch.empty_like(q)
    mode = 1 if ratio == 4 else (2 if ratio else 0)
    pt = fb.page_table
    if nsplit <= 0:
        nsplit = attention_splits(t, h, mode, ratio, topk_idx.shape[1] if mode == 1 else 0, window,
                                  int(fb.max_context), bool(getattr(fb, "is_prefill", False)), num_sms(q.device))
    acc = ml = cnt = None
    if nsplit > 1:
        acc = torch.empty(t, nsplit, h, d, dtype=torch.float32, device=q.device)
        ml = torch.empty(t, nsplit, h, 2, dtype=torch.float32, device=q.device)
        key = q.device.index or 0
        cnt = _ATTN_COUNTERS.get(key)
        if cnt is None or cnt.shape[0] < t:
            cnt = torch.zeros(max(t, 4096), dtype=torch.int32, device=q.device)
            _ATTN_COUNTERS[key] = cnt
    nv.call("sparse_attention", nv.ptr(q), nv.ptr(o), _i32(fb.slots), _i32(fb.positions), _i32(pt), I(pt.stride(0)),
            nv.ptr(swa_cache), _i32(swa_map), nv.ptr(comp_cache if mode else None),
            nv.ptr(topk_idx if mode == 1 else None), nv.ptr(topk_len if mode == 1 else None),
            I(topk_idx.shape[1] if mode == 1 else 0), I(mode), I(ratio), nv.ptr(sink), F(scale), I(ps), I(window),
            nv.ptr(fb.num_valid), I(t), I(h), I(d), I(1 if out_rope is not None else 0),
            rope_params(out_rope if out_rope is not None else _NO_ROPE), I(nsplit), nv.ptr(acc), nv.ptr(ml),
            nv.ptr(cnt))
    return o


_NO_ROPE = RopeSpec.make(64, 10000.0, 0, 1.0, 32, 1)


# --------------------------------------------------------------------------- MoE
_SCORING = {"sqrtsoftplus": 0, "sigmoid": 1, "softmax": 2}


def moe_gate(y, gate_w, bias, topk, scaling, scoring, tid2eid, token_ids, num_valid=None, gate=None):
    """gate: row-sharded exchange context; the router GEMM then waits for each row block's all-gather flag."""
    from .gemm import gemm_bf16_partials

    # the router weight is bf16 in the checkpoint (its fp32 copy converts back losslessly); the model passes the bf16
    # tensor it keeps next to the fp32 one.  No cache keyed by address here: a later model may reuse the address.
    wb = gate_w if gate_w.dtype == torch.bfloat16 else gate_w.to(torch.bfloat16)
    t, e = y.shape[0], gate_w.shape[0]
    scores = gemm_bf16_partials(y, wb, gate=gate)  # [S, T, E]; the selection kernel adds the splits
    idx = torch.empty(t, topk, dtype=torch.int32, device=y.device)
    wts = torch.empty(t, topk, dtype=torch.float32, device=y.device)
    nv.call("moe_topk", nv.ptr(scores), nv.ptr(bias if tid2eid is None else None), nv.ptr(tid2eid),
            nv.ptr(token_ids), nv.ptr(num_valid), nv.ptr(idx), nv.ptr(wts), I(t), I(e), I(topk), F(scaling),
            I(_SCORING[scoring]), I(scores.shape[0]), L(scores.stride(0)))
    return idx, wts


# MINISGL_MOE_KERNEL=f16 selects the W4A16 kernel that dequantises the experts to fp16 inside the SM (csrc/moe.cu);
# the default feeds the packed FP4 weights and their scales to the block-scaled MMA as they are (csrc/moe_mx.cu).
MOE_KERNEL = _os.environ.get("MINISGL_MOE_KERNEL", "mx")


def block_expert_scales(s: torch.Tensor, gate_up: bool) -> torch.Tensor:
    """e8m0 scale bytes [E, rows, K/32] -> [E, row tiles, K/128, 512]: one 512-byte block per (128 weight rows of a
    work item, 128 K elements), byte (m % 32) * 16 + (m // 32) * 4 + k_block for tile row m -- the arrangement that one
    tcgen05.cp moves into tensor memory for the block-scaled MMA.  gate_up: rows are [gate; up] of 2I rows and tile rt
    holds gate rows [64 rt, 64 rt + 64) on m < 64 and the matching up rows on m >= 64 (csrc/moe_mx.cu)."""
    e, rows, kb = s.shape
    assert s.dtype == torch.uint8 and kb % 4 == 0, (s.dtype, s.shape)
    ch = kb // 4
    if gate_up:
        i = rows // 2
        assert i % 64 == 0
        t = s.view(e, 2, i // 64, 64, ch, 4).permute(0, 2, 4, 1, 3, 5).reshape(e, i // 64, ch, 128, 4)
    else:
        assert rows % 128 == 0
        t = s.view(e, rows // 128, 128, ch, 4).permute(0, 1, 3, 2, 4)
    rt = t.shape[1]
    t = t.reshape(e, rt, ch, 4, 32, 4).permute(0, 1, 2, 4, 3, 5)
    return t.contiguous().view(e, rt, ch, 512)


def pack_expert_weights(w: torch.Tensor, gate_up: bool) -> torch.Tensor:
    """Packed FP4 bytes [E, rows, K/2] -> tiles [E, row tiles, K/128, 128, 64]: the 128 rows x 128 K elements of one
    pipeline stage of the grouped GEMM become 8 KiB of consecutive bytes (csrc/moe_mx.cu explains why).  Row order
    inside a tile as in :func:`block_expert_scales`."""
    e, rows, kb2 = w.shape
    assert w.dtype in (torch.int8, torch.uint8) and kb2 % 64 == 0, (w.dtype, w.shape)
    ch = kb2 // 64
    if gate_up:
        i = rows // 2
        assert i % 64 == 0
        return w.view(e, 2, i // 64, 64, ch, 64).permute(0, 2, 4, 1, 3, 5).reshape(e, i // 64, ch, 128, 64)
    assert rows % 128 == 0
    return w.view(e, rows // 128, 128, ch, 64).permute(0, 1, 3, 2, 4).contiguous()


def prepare_experts(weights: dict, prefix: str) -> None:
    """Load-time step of the block-scaled expert kernel: replaces ``prefix + w13 / s13 / w2 / s2`` in ``weights`` by
    their tiled forms (same bytes, other order), one tensor at a time so that at most one extra copy exists.  Tensors
    that are tiled already are left alone."""
    for name, gate_up in (("w13", True), ("w2", False)):
        if weights[prefix + name].dim() == 3:
            weights[prefix + name] = pack_expert_weights(weights[prefix + name], gate_up)
    for name, gate_up in (("s13", True), ("s2", False)):
        if weights[prefix + name].dim() == 3:
            weights[prefix + name] = block_expert_scales(weights[prefix + name], gate_up)


def _tiled(t: torch.Tensor, fn, gate_up: bool, ndim: int) -> torch.Tensor:
    """Tiled form of an expert tensor: given as such (built at load time), or built once and kept on the tensor object
    itself (a cache keyed by address would outlive the tensor and hit a later one)."""
    if t.dim() == ndim:
        return t
    b = getattr(t, "_dsv4_tiled", None)
    if b is None:
        b = fn(t, gate_up)
        t._dsv4_tiled = b
    return b


def route_tile(routes: int, n_experts: int, kernel: str) -> int:
    """Routes per tile of the grouped GEMM (its N dimension): wide enough that an expert's routes rarely need a second
    tile (which would stream the expert's weights again), no wider (the route rows of a tile are loaded per stage)."""
    avg = routes / max(n_experts, 1)
    if kernel != "mx":
        return 32 if avg <= 32 else 64
    return 8 if avg <= 3.5 else 16 if avg <= 7 else 32 if avg <= 16 else 64


@tensors(y="bf16[T,H]", idx="i32[T,K]", w="f32[T,K]")
def moe_routed(y, idx, w, w13, s13, w2, s2, limit, expert_base: int = 0, n_experts: int = 0):
    """Returns (route_rows bf16 [T*topk, H], plan int32, max_tiles) for :func:`moe_finalize`.  Expert tensors in the
    checkpoint layout (w [E, rows, K/2] packed FP4, s [E, rows, K/32] e8m0 bytes) or, for the block-scaled kernel,
    already tiled (:func:`prepare_experts`).  n_experts: experts of the whole layer (default: the resident ones)."""
    t, h = y.shape
    topk = idx.shape[1]
    routes = t * topk
    e_local = w13.shape[0]
    inter = w13.shape[1] * 64 if w13.dim() == 5 else w13.shape[1] // 2
    for a in (w13, s13, w2, s2):
        assert a.is_cuda and a.is_contiguous() and a.dtype in (torch.int8, torch.uint8) and a.shape[0] == e_local
    nt = route_tile(routes, n_experts or e_local, MOE_KERNEL)
    max_tiles = min(e_local, routes) + routes // nt + 1
    plan = torch.empty(4 + 3 * max_tiles + 3 * routes, dtype=torch.int32, device=y.device)
    nv.call("moe_plan", nv.ptr(idx), nv.ptr(w), I(routes), I(e_local), I(expert_base), I(nt), nv.ptr(plan),
            I(max_tiles))
    sms = num_sms(y.device)
    rows = torch.empty(routes, h, dtype=y.dtype, device=y.device)
    if MOE_KERNEL == "mx":
        w13, w2 = _tiled(w13, pack_expert_weights, True, 5), _tiled(w2, pack_expert_weights, False, 5)
        b13, b2 = _tiled(s13, block_expert_scales, True, 4), _tiled(s2, block_expert_scales, False, 4)
        u8 = dict(dtype=torch.uint8, device=y.device)
        # rows 2 pos / 2 pos + 1: hi / lo of a route; one 512-byte scale block per (route tile, 128 K elements)
        xq, sfx = torch.empty(2 * routes, h, **u8), torch.empty(max_tiles, h // 128, 512, **u8)
        nv.call("moe_mx_permute", nv.ptr(y), nv.ptr(xq), nv.ptr(sfx), nv.ptr(plan), I(routes), I(max_tiles), I(topk),
                I(h), I(nt))
        act, sfa = torch.empty(2 * routes, inter, **u8), torch.empty(max_tiles, inter // 128, 512, **u8)
        nv.call("moe_mx_gemm", I(1), I(nt), nv.ptr(w13), nv.ptr(b13), nv.ptr(xq), nv.ptr(sfx), nv.ptr(plan),
                I(routes), I(max_tiles), nv.ptr(act), nv.ptr(sfa), I(e_local), I(h), I(inter), I(inter),
                F(limit or 0.0), I(sms))
        nv.call("moe_mx_gemm", I(2), I(nt), nv.ptr(w2), nv.ptr(b2), nv.ptr(act), nv.ptr(sfa), nv.ptr(plan),
                I(routes), I(max_tiles), nv.ptr(rows), nv.ptr(None), I(e_local), I(inter), I(h), I(h), F(0.0), I(sms))
        return rows, plan, max_tiles
    assert w13.dim() == 3 and s13.dim() == 3, "the fp16 expert kernel reads the checkpoint layout"
    xs = torch.empty(routes, h, dtype=torch.float16, device=y.device)
    nv.call("moe_permute", nv.ptr(y), nv.ptr(xs), nv.ptr(plan), I(routes), I(max_tiles), I(topk), I(h))
    act = torch.empty(routes, inter, dtype=torch.float16, device=y.device)
    nv.call("moe_gemm", I(1), I(nt), nv.ptr(w13), nv.ptr(s13), nv.ptr(xs), I(routes), nv.ptr(plan), I(routes),
            I(max_tiles), nv.ptr(act), I(e_local), I(h), I(inter), I(inter), F(limit or 0.0), I(sms))
    nv.call("moe_gemm", I(2), I(nt), nv.ptr(w2), nv.ptr(s2), nv.ptr(act), I(routes), nv.ptr(plan), I(routes),
            I(max_tiles), nv.ptr(rows), I(e_local), I(inter), I(h), I(h), F(0.0), I(sms))
    return rows, plan, max_tiles


def moe_finalize(rows, plan, max_tiles, shared, num_valid, t, topk, h, hc=None):
    """hc = (residual [t,4,h], post, comb): returns the new residual streams (post mix fused), else the layer output."""
    if hc is not None:
        res, post, comb = hc
        xout = torch.empty_like(res)
        nv.call("moe_finalize", nv.ptr(rows), nv.ptr(plan), I(t * topk), I(max_tiles), nv.ptr(shared), nv.ptr(None),
                nv.ptr(num_valid), I(t), I(topk), I(h), nv.ptr(res), nv.ptr(post), nv.ptr(comb), nv.ptr(xout))
        return xout
    out = torch.empty(t, h, dtype=rows.dtype, device=rows.device)
    nv.call("moe_finalize", nv.ptr(rows), nv.ptr(plan), I(t * topk), I(max_tiles), nv.ptr(shared), nv.ptr(out),
            nv.ptr(num_valid), I(t), I(topk), I(h), nv.ptr(None), nv.ptr(None), nv.ptr(None), nv.ptr(None))
    return out


def moe_experts(y, idx, w, w13, s13, w2, s2, limit, expert_base: int = 0):
    rows, plan, max_tiles = moe_routed(y, idx, w, w13, s13, w2, s2, limit, expert_base)
    return moe_finalize(rows, plan, max_tiles, None, None, y.shape[0], idx.shape[1], y.shape[1])


# --------------------------------------------------------------------------- sampling
@tensors(logits="f32[_,_]")
def argmax(logits):
    b, v = logits.shape
    out = torch.empty(b, dtype=torch.int64, device=logits.device)
    nv.call("argmax", nv.ptr(logits), nv.ptr(out), I(b), I(v))
    return out


@tensors(logits="f32[B,_]", temperature="f32[B]", top_k="i32[B]", top_p="f32[B]", uniform="f32[B]", mask_ids="?i32[B,_]")
def sample(logits, temperature, top_k, top_p, uniform, mask_ids=None):
    b, v = logits.shape
    out = torch.empty(b, dtype=torch.int64, device=logits.device)
    n_mask = 0 if mask_ids is None else mask_ids.shape[1]
    nv.call("sample", nv.ptr(logits), I(b), I(v), nv.ptr(temperature), nv.ptr(top_k), nv.ptr(top_p), nv.ptr(uniform),
            nv.ptr(mask_ids), I(n_mask), nv.ptr(out))
    return out
