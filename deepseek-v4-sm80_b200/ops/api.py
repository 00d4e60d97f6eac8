"""Operator facade used by the model.

Each function has two bodies: CUDA tensors go to the hand-written sm_100a kernels (``ops/cuda.py`` ->
``libdsv4_b200.so``), CPU tensors to the PyTorch oracle in ``ops/ref.py``.  There is no third path: a CUDA
tensor never falls back to PyTorch silently (``cuda.py`` raises when the library is missing).
"""
from __future__ import annotations

import torch

from . import gemm as _gemm
from . import ref

gemm_bf16 = _gemm.gemm_bf16
gemm_fp8 = _gemm.gemm_fp8
gemm_bf16_grouped = _gemm.gemm_bf16_grouped


def _cu():
    from . import cuda

    return cuda


# --------------------------------------------------------------------------- page-table helpers (CPU path)
def _locs(fb, pos):
    """Token locations of (row slot, position) pairs; pos [T,n] may be negative (-> -1)."""
    p = pos.clamp_min(0).long()
    loc = fb.page_table[fb.slots.long()[:, None], p]
    return torch.where(pos >= 0, loc, torch.full_like(loc, -1))


def swa_rows(fb, swa_map, ps: int, window: int):
    off = torch.arange(window - 1, -1, -1, device=fb.positions.device)
    pos = fb.positions.long()[:, None] - off[None, :]
    loc = _locs(fb, pos).long()
    slot = swa_map[(loc.clamp_min(0) // ps)].long()
    row = slot * ps + loc.clamp_min(0) % ps
    return torch.where((loc >= 0) & (slot >= 0), row, torch.full_like(row, -1))


def comp_rows_all(fb, ps: int, ratio: int, width: int):
    j = torch.arange(width, device=fb.positions.device)[None, :]
    n = ((fb.positions.long() + 1) // ratio)[:, None]
    loc = _locs(fb, torch.where(j < n, j * ratio + ratio - 1, torch.full_like(j, -1))).long()
    return torch.where(loc >= 0, ref.comp_row(loc.clamp_min(0), ps, ratio), torch.full_like(loc, -1))


def comp_rows_from_idx(fb, idx, ps: int, ratio: int):
    loc = _locs(fb, torch.where(idx >= 0, idx.long() * ratio + ratio - 1, torch.full_like(idx.long(), -1))).long()
    return torch.where(loc >= 0, ref.comp_row(loc.clamp_min(0), ps, ratio), torch.full_like(loc, -1))


# --------------------------------------------------------------------------- index audit (MINISGL_DEBUG_BOUNDS=1)
INDEX_TAGS = {"input_ids": 1, "positions": 2, "slots": 3, "out_loc": 4, "page_table": 5, "expert_ids": 6,
              "indexer_topk": 7}


def check_index(idx, lo: int, hi: int, what: str) -> None:
    """Every entry of ``idx`` must lie in [lo, hi).  CUDA: a device kernel records a violation in the status word
    (no synchronisation; ``native.assert_device_ok()`` raises it); CPU: raises at once."""
    if idx.is_cuda:
        return _cu().check_index(idx.contiguous(), lo, hi, INDEX_TAGS[what])
    if idx.numel() and (int(idx.min()) < lo or int(idx.max()) >= hi):
        raise IndexError(f"{what}: index outside [{lo}, {hi})")


# --------------------------------------------------------------------------- elementwise
def embed(ids, weight, m: int, feedback=None, slots=None):
    """feedback [slots+1] int32 / slots [T]: row t embeds the token ``feedback[slots[t]]`` (the previous step's sample,
    kept on the device) and stores it into ``ids[t]``."""
    if ids.is_cuda:
        return _cu().embed(ids, weight, m, feedback, slots)
    if feedback is not None:
        ids.copy_(feedback[slots.long()])
    return weight[ids.long()].unsqueeze(1).repeat(1, m, 1)


def greedy_tokens(logits, v_base: int, slots, num_valid, token_feedback, out=None, comm_ctx=None):
    """Greedy sample of every row (lowest index wins ties) into ``out`` [rows] int32 and, for valid rows, into
    ``token_feedback[slots[row]]``.  ``logits`` may be one rank's vocabulary shard (first column = token v_base)."""
    if logits.is_cuda:
        return _cu().greedy_tokens(logits, v_base, slots, num_valid, token_feedback, out, comm_ctx)
    tok = (logits.float().argmax(-1) + v_base).to(torch.int32)
    if out is None:
        out = torch.empty_like(tok)
    out.copy_(tok)
    n = logits.shape[0] if num_valid is None else int(num_valid)
    token_feedback[slots[:n].long()] = tok[:n]
    return out


def rms_norm(x, weight, eps: float, want_q: bool = False):
    """want_q: returns (out, (e4m3, scales)) -- on CUDA the normalising kernel writes the quantisation too."""
    if x.is_cuda:
        return _cu().rms_norm(x, weight, eps, want_q)
    out = ref.rms_norm(x, weight, eps)
    return (out, fp8_quant(out)) if want_q else out


def fp8_quant(x, block: int = 128):
    if x.is_cuda:
        return _cu().fp8_quant(x, block)
    from . import quant

    return quant.fp8_act_quant(x.contiguous(), block)


def silu_mul_clamp(gate_up, limit):
    if gate_up.is_cuda:
        return _cu().silu_mul_clamp(gate_up, limit)
    return ref.silu_mul_clamp(gate_up, limit)


def silu_mul_clamp_quant(gate_up, limit):
    """(e4m3, scales) of the SwiGLU activation (one kernel on CUDA)."""
    if gate_up.is_cuda:
        return _cu().silu_mul_clamp_quant(gate_up, limit)
    return fp8_quant(ref.silu_mul_clamp(gate_up, limit))


def add_cast(routed, shared, num_valid=None):
    if routed.is_cuda:
        return _cu().add_cast(routed, shared, num_valid)
    out = (routed.float() + shared.float()).to(routed.dtype)
    if num_valid is not None:
        out[int(num_valid):] = 0
    return out


def rope_tail(x, positions, spec, inverse: bool = False):
    if x.is_cuda:
        return _cu().rope_tail(x, positions, spec, inverse)
    return ref.rope_tail(x, positions, spec, inverse).to(x.dtype)


def q_kv_norm_rope_store(q, kv, positions, kv_w, eps, spec, swa_cache, out_loc, swa_map, ps: int, qat: bool):
    if q.is_cuda:
        return _cu().q_kv_norm_rope_store(q, kv, positions, kv_w, eps, spec, swa_cache, out_loc, swa_map, ps, qat)
    qo, ko = ref.q_kv_norm_rope(q, kv, positions, kv_w, eps, spec, qat)
    loc = out_loc.long()
    slot = swa_map[loc.clamp_min(0) // ps].long()
    ok = (loc >= 0) & (slot >= 0)
    swa_cache[(slot * ps + loc % ps)[ok]] = ko[ok]
    return qo, ko


# --------------------------------------------------------------------------- hyper-connections
def hc_pre(x, fn, scale, base, iters, eps, norm_eps, norm_w=None, want_q: bool = False, out=None):
    """Returns (y, post, comb); with ``norm_w`` y is additionally RMS-normalised (fused on CUDA); with ``want_q``
    a fourth item, the (e4m3, scales) quantisation of y (also fused on CUDA).  ``out`` (CUDA only): result rows
    (y, q, s) to write into."""
    if x.is_cuda:
        return _cu().hc_pre(x, fn, scale, base, iters, eps, norm_eps, norm_w, want_q, out)
    y, post, comb = ref.hc_pre(x, fn, scale, base, iters, eps, norm_eps)
    if norm_w is not None:
        y = ref.rms_norm(y, norm_w, norm_eps)
    return (y, post, comb, fp8_quant(y)) if want_q else (y, post, comb)


def hc_post(y, residual, post, comb):
    if y.is_cuda:
        return _cu().hc_post(y, residual, post, comb)
    return ref.hc_post(y, residual, post, comb)


def hc_head(x, fn, scale, base, eps, norm_eps, norm_w=None):
    if x.is_cuda:
        return _cu().hc_head(x, fn, scale, base, eps, norm_eps, norm_w)
    y = ref.hc_head(x, fn, scale, base, eps, norm_eps)
    return ref.rms_norm(y, norm_w, norm_eps) if norm_w is not None else y


# --------------------------------------------------------------------------- compressors
def compress(proj, fb, ratio: int, d: int, ape, ring, ckpt, ps: int):
    """Pools group boundaries of this call and then carries the call's rows into the ring / checkpoint state."""
    if proj.is_cuda:
        return _cu().compress(proj, fb, ratio, d, ape, ring, ckpt, ps)
    pooled = ref.compress_pool(proj, fb.positions, fb.slots, ratio, d, ape, ring, ckpt, fb.page_table, ps)
    ref.compress_state_store(proj, fb.positions, fb.slots, ratio, d, ape, ring, ckpt, fb.page_table, ps)
    return pooled


def compress_store(pooled, fb, norm_w, eps, spec, cache, ps: int, ratio: int):
    if pooled.is_cuda:
        return _cu().compress_store(pooled, fb, norm_w, eps, spec, cache, ps, ratio)
    ok = ((fb.positions.long() + 1) % ratio == 0) & (fb.out_loc >= 0)
    if bool(ok.any()):
        y = ref.compress_norm_rope(pooled[ok], fb.positions[ok].long(), norm_w, eps, spec, ratio)
        cache[ref.comp_row(fb.out_loc[ok].long(), ps, ratio)] = y


def indexer_q_encode(q, weights, positions, spec, softmax_scale, head_scale):
    if q.is_cuda:
        return _cu().indexer_q_encode(q, weights, positions, spec, softmax_scale, head_scale)
    return ref.indexer_q_encode(q, weights, positions, spec, softmax_scale, head_scale)


def indexer_kv_store(pooled, fb, norm_w, eps, spec, vals, scales, ps: int):
    if pooled.is_cuda:
        return _cu().indexer_kv_store(pooled, fb, norm_w, eps, spec, vals, scales, ps)
    ok = ((fb.positions.long() + 1) % 4 == 0) & (fb.out_loc >= 0)
    if bool(ok.any()):
        codes, sc = ref.indexer_kv_encode(pooled[ok], fb.positions[ok].long(), norm_w, eps, spec)
        rows = ref.comp_row(fb.out_loc[ok].long(), ps, 4)
        vals[rows] = codes
        scales[rows] = sc


def indexer_select(qc, wf, vals, scales, fb, ps: int, k: int):
    """Top-k compressed entries per token: (idx int32 [T,k] of compressed indices j, -1 padded; len int32 [T])."""
    if qc.is_cuda:
        return _cu().indexer_select(qc, wf, vals, scales, fb, ps, k)
    width = max(fb.max_context // 4, 1)
    rows = comp_rows_all(fb, ps, 4, width)
    lens = ((fb.positions.long() + 1) // 4).to(torch.int32)
    logits = ref.indexer_logits(qc, wf, vals, scales, rows, lens)
    return ref.topk_select(logits, lens, k)


# --------------------------------------------------------------------------- attention
def attention(q, fb, swa_cache, swa_map, comp_cache, ratio: int, topk_idx, topk_len, sink, scale, ps: int,
              window: int, out_rope=None):
    """``out_rope``: also rotate the last ``rotary_dim`` dims of every output row by minus its position (fused into
    the kernel's epilogue on CUDA, :func:`rope_tail` with ``inverse=True`` on the oracle path)."""
    if q.is_cuda:
        return _cu().attention(q, fb, swa_cache, swa_map, comp_cache, ratio, topk_idx, topk_len, sink, scale, ps,
                               window, out_rope)
    srows = swa_rows(fb, swa_map, ps, window)
    crows = None
    if ratio == 4:
        idx = torch.where((topk_len > 0)[:, None], topk_idx, torch.full_like(topk_idx, -1))
        crows = comp_rows_from_idx(fb, idx, ps, 4)
    elif ratio:
        crows = comp_rows_all(fb, ps, ratio, max(fb.max_context // ratio, 1))
    o = ref.sparse_attention(q, comp_cache, crows, swa_cache, srows, sink, scale)
    return rope_tail(o, fb.positions, out_rope, inverse=True) if out_rope is not None else o


# --------------------------------------------------------------------------- MoE
def moe_gate(y, gate_w, bias, topk, scaling, scoring, tid2eid, token_ids, num_valid=None, gate=None):
    if y.is_cuda:
        return _cu().moe_gate(y, gate_w, bias, topk, scaling, scoring, tid2eid, token_ids, num_valid, gate)
    idx, w = ref.moe_gate(y, gate_w, bias, topk, scaling, scoring, tid2eid, token_ids)
    if num_valid is not None:
        idx[int(num_valid):] = -1
        w[int(num_valid):] = 0
    return idx, w


def moe_experts(y, idx, w, w13, s13, w2, s2, limit, expert_base: int = 0):
    if y.is_cuda:
        return _cu().moe_experts(y, idx, w, w13, s13, w2, s2, limit, expert_base)
    e_local = w13.shape[0]
    local = idx - expert_base
    local = torch.where((local >= 0) & (local < e_local) & (idx >= 0), local, torch.full_like(local, -1))
    return ref.moe_experts(y, local, w, w13, s13, w2, s2, limit)


# --------------------------------------------------------------------------- sampling
def sample(logits, temperature, top_k, top_p, uniform, mask_ids=None):
    if logits.is_cuda:
        return _cu().sample(logits, temperature, top_k, top_p, uniform, mask_ids)
    return ref.sample(logits, temperature, top_k, top_p, uniform, mask_ids)


def argmax(logits):
    if logits.is_cuda:
        return _cu().argmax(logits)
    return logits.argmax(-1)
