"""Plain-PyTorch statement of every operator of the DeepSeek-V4 forward pass.

This module is the oracle: the CPU model runs on it, and every CUDA kernel is
tested against it.  The math follows the reference's release path
(python/minisgl/kernel/triton/deepseek_v4.py and
debug/dsv4/kernel/deepseek_v4_reference.py); citations are given per function.
All functions work on any device and compute in fp32 unless stated otherwise.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import quant


# --------------------------------------------------------------------------- RoPE
@dataclass(frozen=True)
class RopeSpec:
    """Interleaved-pair rotary embedding on the last ``rotary_dim`` dims with an optional YaRN ramp
    (kernel/triton/deepseek_v4.py:97-141 and :1807-1827)."""

    rotary_dim: int
    base: float
    use_scaling: bool = False
    factor: float = 1.0
    low: int = 0
    high: int = 0

    @staticmethod
    def make(rotary_dim, base, original_seq_len=0, factor=1.0, beta_fast=32, beta_slow=1) -> "RopeSpec":
        if original_seq_len <= 0:
            return RopeSpec(rotary_dim, float(base))

        def corr(nrot):
            return rotary_dim * math.log(original_seq_len / (nrot * 2 * math.pi)) / (2 * math.log(base))

        low = max(math.floor(corr(beta_fast)), 0)
        high = min(math.ceil(corr(beta_slow)), rotary_dim // 2 - 1)
        return RopeSpec(rotary_dim, float(base), True, float(factor), int(low), int(high))

    @property
    def scale_denom(self) -> float:
        return float(max(self.high - self.low, 1))


def rope_cos_sin(positions: torch.Tensor, spec: RopeSpec, inverse: bool = False):
    half = spec.rotary_dim // 2
    i = torch.arange(half, dtype=torch.float32, device=positions.device)
    inv = torch.exp(-(2.0 * i / spec.rotary_dim) * math.log(spec.base))
    if spec.use_scaling:
        ramp = ((i - spec.low) / spec.scale_denom).clamp(0.0, 1.0)
        smooth = 1.0 - ramp
        inv = inv / spec.factor * (1.0 - smooth) + inv * smooth
    theta = positions.float()[:, None] * inv[None, :]
    if inverse:
        theta = -theta
    theta = theta - torch.floor((theta + math.pi) / (2 * math.pi)) * (2 * math.pi)
    return torch.cos(theta), torch.sin(theta)


def rope_tail(x: torch.Tensor, positions: torch.Tensor, spec: RopeSpec, inverse: bool = False) -> torch.Tensor:
    """x [T, ..., D] (any dtype) -> fp32 with the last rotary_dim dims rotated at positions [T]."""
    xf = x.float().clone()
    cos, sin = rope_cos_sin(positions, spec, inverse)
    while cos.dim() < xf.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    tail = xf[..., -spec.rotary_dim:]
    a, b = tail[..., 0::2], tail[..., 1::2]
    ra, rb = a * cos - b * sin, a * sin + b * cos
    xf[..., -spec.rotary_dim:] = torch.stack((ra, rb), dim=-1).flatten(-2)
    return xf


# --------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def swa_qat(x_bf16: torch.Tensor, nope_dim: int, block: int = 64) -> torch.Tensor:
    """Block-64 power-of-two e4m3 quantise-dequantise of the first ``nope_dim`` dims
    (kernel/triton/deepseek_v4.py:266-276)."""
    out = x_bf16.clone()
    out[..., :nope_dim] = quant.fp8_fake_quant(x_bf16[..., :nope_dim].contiguous(), block)
    return out


def q_kv_norm_rope(q, kv, positions, kv_norm_w, eps, spec: RopeSpec, qat: bool = True):
    """q [T,H,D]: weightless per-head RMSNorm + RoPE.  kv [T,D]: RMSNorm(w) + RoPE + SWA QAT.
    Returns (q, kv) in the input dtype (kernel/triton/deepseek_v4.py:143-280)."""
    qf = q.float()
    qn = qf * torch.rsqrt(qf.square().mean(-1, keepdim=True) + eps)
    qo = rope_tail(qn, positions, spec).to(q.dtype)
    kf = kv.float()
    kn = kf * torch.rsqrt(kf.square().mean(-1, keepdim=True) + eps) * kv_norm_w.float()
    ko = rope_tail(kn, positions, spec).to(kv.dtype)
    if qat:
        ko = swa_qat(ko, kv.shape[-1] - spec.rotary_dim)
    return qo, ko


# --------------------------------------------------------------------------- hyper-connections
def hc_pre(x, fn, scale, base, iters: int, eps: float, norm_eps: float):
    """x [T,m,H] bf16 residual streams -> (y [T,H] bf16, post [T,m] f32, comb [T,m,m] f32)
    (kernel/triton/deepseek_v4.py:773-923; host :3765).  ``fn`` is [(2+m)m, m*H]."""
    t, m, h = x.shape
    flat = x.reshape(t, m * h)
    mixes = flat.to(torch.bfloat16).float() @ fn.to(torch.bfloat16).float().t()
    xf = x.float()
    r = torch.rsqrt(xf.reshape(t, -1).square().mean(-1, keepdim=True) + norm_eps)
    sc = scale.float()
    b = base.float()
    pre = torch.sigmoid(mixes[:, :m] * r * sc[0] + b[:m]) + eps
    post = 2.0 * torch.sigmoid(mixes[:, m:2 * m] * r * sc[1] + b[m:2 * m])
    logits = (mixes[:, 2 * m:] * r * sc[2] + b[2 * m:]).reshape(t, m, m)
    e = torch.exp(logits - logits.amax(-1, keepdim=True))
    comb = e / e.sum(-1, keepdim=True).clamp_min(eps) + eps
    comb = comb / (comb.sum(1, keepdim=True) + eps)
    for _ in range(max(iters - 1, 0)):
        comb = comb / (comb.sum(2, keepdim=True) + eps)
        comb = comb / (comb.sum(1, keepdim=True) + eps)
    y = (pre[:, :, None] * xf).sum(1).to(x.dtype)
    return y, post, comb


def hc_post(y, residual, post, comb):
    """out[t,i] = post[t,i]*y[t] + sum_j comb[t,j,i]*residual[t,j]  (kernel/triton/deepseek_v4.py:720-769)."""
    out = post.float()[:, :, None] * y.float()[:, None, :]
    out = out + torch.einsum("tji,tjh->tih", comb.float(), residual.float())
    return out.to(residual.dtype)


def hc_head(x, fn, scale, base, eps: float, norm_eps: float):
    """Collapse the m streams: y = sum_i (sigmoid(mix_i*r*s+b_i)+eps) x_i  (kernel/triton/deepseek_v4.py:860-923)."""
    t, m, h = x.shape
    mixes = x.reshape(t, m * h).to(torch.bfloat16).float() @ fn.to(torch.bfloat16).float().t()
    xf = x.float()
    r = torch.rsqrt(xf.reshape(t, -1).square().mean(-1, keepdim=True) + norm_eps)
    pre = torch.sigmoid(mixes * r * scale.float()[0] + base.float()) + eps
    return (pre[:, :, None] * xf).sum(1).to(x.dtype)


def silu_mul_clamp(gate_up: torch.Tensor, limit) -> torch.Tensor:
    """[.., 2I] -> [.., I]: silu(min(g, L)) * clamp(u, -L, L) in fp32 (kernel/triton/deepseek_v4.py:43-73)."""
    g, u = gate_up.float().chunk(2, dim=-1)
    if limit is not None and limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
    return (F.silu(g) * u).to(gate_up.dtype)


# --------------------------------------------------------------------------- paged-cache addressing
def comp_row(loc: torch.Tensor, page_size: int, ratio: int) -> torch.Tensor:
    """Cache row of the compressed entry whose last source token lives at token location ``loc``.
    A page of ``page_size`` tokens owns ``max(page_size // ratio, 1)`` compressed rows."""
    rpp = max(page_size // ratio, 1)
    return (loc // page_size) * rpp + (loc % page_size) // ratio


# --------------------------------------------------------------------------- compressors
def compress_pool(proj, positions, slots, ratio: int, d: int, ape, ring, ckpt, page_table, page_size: int):
    """Softmax pooling of the KV compressor at group boundaries ((pos+1) % ratio == 0).

    proj [T, W] fp32 is ``x @ wkv_gate^T``: W = 4d for ratio 4 ([kv_l | kv_r | score_l | score_r],
    overlap compressor) and 2d otherwise ([kv | score]).  Source rows come from this call when the
    (slot, position) matches, else from the per-request ring (``ring[slot*L + pos%L]``, L = 8 for
    ratio 4 else ratio) or, for the older half of a ratio-4 group that lies in the previous page,
    from that page's 4-row checkpoint.  Returns pooled [T, d] fp32 (zero on non-boundary rows).
    Mirrors kernel/triton/deepseek_v4.py:2419-2622 (C4) and :2833-2917 (C128).
    """
    t = proj.shape[0]
    out = torch.zeros(t, d, dtype=torch.float32, device=proj.device)
    pos_l = positions.tolist()
    slot_l = slots.tolist()
    index = {(slot_l[i], pos_l[i]): i for i in range(t)}
    apef = ape.float()
    for r in range(t):
        p, s = pos_l[r], slot_l[r]
        if (p + 1) % ratio != 0:
            continue
        kvs, scs = [], []
        if ratio == 4:
            for src in range(8):
                lp = p - (7 - src)
                right = src >= 4
                if lp < 0:
                    continue
                cur = index.get((s, lp))
                ko, so = (d, 3 * d) if right else (0, 2 * d)
                if cur is not None:
                    kv, sc = proj[cur, ko:ko + d], proj[cur, so:so + d]
                elif (not right) and lp // page_size != p // page_size:
                    page = int(page_table[s, lp]) // page_size
                    row = ckpt[page * 4 + lp % 4]
                    kv, sc = row[:d], row[d:2 * d]
                else:
                    row = ring[s * 8 + lp % 8]
                    kv, sc = row[ko:ko + d], row[so:so + d]
                a = apef[src % 4, (d if right else 0):(2 * d if right else d)]
                kvs.append(kv.float())
                scs.append(sc.float() + a)
        else:
            for src in range(ratio):
                lp = p - (ratio - 1 - src)
                if lp < 0:
                    continue
                cur = index.get((s, lp))
                if cur is not None:
                    kvs.append(proj[cur, :d].float())
                    scs.append(proj[cur, d:2 * d].float() + apef[src])
                else:
                    row = ring[s * ratio + src]
                    kvs.append(row[:d].float())
                    scs.append(row[d:2 * d].float())
        kv = torch.stack(kvs)
        sc = torch.stack(scs)
        w = torch.exp(sc - sc.amax(0, keepdim=True))
        out[r] = (kv * w).sum(0) / w.sum(0)
    return out


def compress_state_store(proj, positions, slots, ratio: int, d: int, ape, ring, ckpt, page_table, page_size: int):
    """Carries this call's projected rows to later calls: writes the per-request ring (last writer per
    ring slot wins) and, for ratio 4, the left halves of the last four tokens of every page into the
    page checkpoint.  For ratio != 4 the ring row holds [kv | score + ape[pos % ratio]].
    Mirrors kernel/triton/deepseek_v4.py:2631-2716 and :2921-2975."""
    t = proj.shape[0]
    pos_l = positions.tolist()
    slot_l = slots.tolist()
    ring_len = 8 if ratio == 4 else ratio
    for r in range(t):
        p, s = pos_l[r], slot_l[r]
        later = r + ring_len
        if later < t and slot_l[later] == s and pos_l[later] == p + ring_len:
            pass
        elif ratio == 4:
            ring[s * 8 + p % 8] = proj[r]
        else:
            row = proj[r].clone()
            row[d:2 * d] += ape.float()[p % ratio]
            ring[s * ratio + p % ratio] = row
        if ratio == 4 and p % page_size >= page_size - 4:
            page = int(page_table[s, p]) // page_size
            ckpt[page * 4 + p % 4, :d] = proj[r, :d]
            ckpt[page * 4 + p % 4, d:2 * d] = proj[r, 2 * d:3 * d]


def compress_norm_rope(pooled, positions, weight, eps, spec: RopeSpec, ratio: int):
    """pooled fp32 -> bf16 -> RMSNorm(weight) -> RoPE at position pos+1-ratio -> bf16
    (kernel/triton/deepseek_v4.py:282-362)."""
    pb = pooled.to(torch.bfloat16).float()
    y = pb * torch.rsqrt(pb.square().mean(-1, keepdim=True) + eps) * weight.float()
    return rope_tail(y, positions + 1 - ratio, spec).to(torch.bfloat16)


# --------------------------------------------------------------------------- indexer
def hadamard128(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised 128-point Walsh-Hadamard transform along the last dim (7 butterfly stages)."""
    y = x.float()
    n = y.shape[-1]
    h = 1
    while h < n:
        y = y.reshape(*y.shape[:-1], n // (2 * h), 2, h)
        y = torch.stack((y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]), dim=-2)
        y = y.reshape(*y.shape[:-3], n)
        h *= 2
    return y


def indexer_kv_encode(pooled, positions, weight, eps, spec: RopeSpec):
    """Indexer key row: bf16 -> RMSNorm(fp32 weight) -> bf16 -> RoPE at pos-3 -> bf16 -> Hadamard * 128^-1/2
    -> bf16 -> power-of-two e4m3.  Returns (codes uint8 [T,128], scale fp32 [T])
    (kernel/triton/deepseek_v4.py:1188-1267; csrc/jit/dsv4_c4_indexer_rmsnorm_bf16.cu:45-85)."""
    pb = pooled.to(torch.bfloat16).float()
    y = (pb * torch.rsqrt(pb.square().mean(-1, keepdim=True) + eps) * weight.float()).to(torch.bfloat16)
    y = rope_tail(y, positions - 3, spec).to(torch.bfloat16)
    y = (hadamard128(y) * (128 ** -0.5)).to(torch.bfloat16).float()
    scale = quant.pow2_scale(y.abs().amax(-1, keepdim=True))
    q = (y / scale).clamp(-448, 448).to(quant.FP8)
    return q.view(torch.uint8), scale.squeeze(-1)


def indexer_q_encode(q, weights, positions, spec: RopeSpec, softmax_scale: float, head_scale: float):
    """q [T,Hi,128] bf16 -> RoPE -> per-(token, head) power-of-two e4m3; the scale is folded into the
    per-head weight: w' = w * scale * softmax_scale * head_scale  (kernel/triton/deepseek_v4.py:1095-1136)."""
    qr = rope_tail(q, positions, spec).to(torch.bfloat16).float()
    scale = quant.pow2_scale(qr.abs().amax(-1, keepdim=True))
    qq = (qr / scale).clamp(-448, 448).to(quant.FP8)
    wf = weights.float() * scale.squeeze(-1) * softmax_scale * head_scale
    return qq.view(torch.uint8), wf


def indexer_logits(q_codes, w_folded, k_codes, k_scale, rows, lens):
    """logit[t, j] = sum_h relu(q[t,h] . k[rows[t,j]]) * w[t,h] * k_scale  for j < lens[t], else -inf.
    rows [T, J] are indexer-cache rows (kernel/triton/deepseek_v4.py:1296-1384)."""
    t, jmax = rows.shape
    q = q_codes.view(quant.FP8).float()                      # [T,H,128]
    k = k_codes.view(quant.FP8).float()[rows.clamp_min(0).long()]  # [T,J,128]
    ks = k_scale[rows.clamp_min(0).long()]                   # [T,J]
    s = torch.einsum("thd,tjd->thj", q, k)
    logit = (torch.relu(s) * w_folded[:, :, None]).sum(1) * ks
    j = torch.arange(jmax, device=rows.device)[None, :]
    return torch.where(j < lens[:, None], logit, torch.full_like(logit, float("-inf")))


def topk_select(logits, lens, k: int):
    """Per row: indices of the k largest of logits[:len] ordered by (score desc, index asc); rows with
    len <= k keep 0..len-1; a non-finite score inside the valid range invalidates the row (len -1).
    Returns (idx int32 [T,k] padded with -1, out_len int32 [T])  (csrc/jit/dsv4_topk_v1.cu:275-479)."""
    t = logits.shape[0]
    idx = torch.full((t, k), -1, dtype=torch.int32, device=logits.device)
    out_len = torch.zeros(t, dtype=torch.int32, device=logits.device)
    for r in range(t):
        n = int(lens[r])
        if n <= 0:
            continue
        row = logits[r, :n].float()
        if n <= k:
            idx[r, :n] = torch.arange(n, dtype=torch.int32, device=logits.device)
            out_len[r] = n
            continue
        if not bool(torch.isfinite(row).all()):
            out_len[r] = -1
            continue
        order = sorted(range(n), key=lambda i: (-float(row[i]), i))[:k]
        idx[r] = torch.tensor(order, dtype=torch.int32, device=logits.device)
        out_len[r] = k
    return idx, out_len


# --------------------------------------------------------------------------- attention
def sparse_attention(q, comp_cache, comp_rows, swa_cache, swa_rows, sink, scale: float):
    """Per token and head: softmax over {sink} U compressed rows U sliding-window rows of scale*q.k, value = the
    same 512-d row; the sink only adds exp(sink - m) to the denominator.  Index -1 = absent.
    q [T,H,D] bf16; *_rows int [T,n]; returns [T,H,D] bf16
    (csrc/jit/dsv4_sparse_attention_two_source_bf16.cu:77-168)."""
    t, h, d = q.shape
    parts, masks = [], []
    if comp_cache is not None and comp_rows is not None and comp_rows.shape[1] > 0:
        parts.append(comp_cache[comp_rows.clamp_min(0).long()].float())
        masks.append(comp_rows >= 0)
    parts.append(swa_cache[swa_rows.clamp_min(0).long()].float())
    masks.append(swa_rows >= 0)
    kv = torch.cat(parts, dim=1)            # [T,n,D]
    mask = torch.cat(masks, dim=1)          # [T,n]
    s = torch.einsum("thd,tnd->thn", q.float(), kv) * scale
    s = s.masked_fill(~mask[:, None, :], float("-inf"))
    m = torch.maximum(s.amax(-1), sink.float()[None, :])
    p = torch.exp(s - m[..., None])
    denom = p.sum(-1) + torch.exp(sink.float()[None, :] - m)
    o = torch.einsum("thn,tnd->thd", p, kv) / denom[..., None]
    return o.to(q.dtype)


# --------------------------------------------------------------------------- MoE
def moe_gate(h, w_gate, bias, topk: int, scaling: float, scoring: str = "sqrtsoftplus", tid2eid=None,
             token_ids=None):
    """Router: fp32 scores -> sqrt(softplus) -> top-k of (p + bias) (or hash lookup) -> weights p/sum * scaling
    (python/minisgl/kernel/deepseek_v4.py:1281-1315)."""
    scores = h.float() @ w_gate.float().t()
    if scoring == "sqrtsoftplus":
        p = torch.sqrt(F.softplus(scores))
    elif scoring == "sigmoid":
        p = torch.sigmoid(scores)
    else:
        p = torch.softmax(scores, dim=-1)
    if tid2eid is not None:
        idx = tid2eid[token_ids.long()].long()
    else:
        sel = p + bias.float() if bias is not None else p
        # ties broken towards the lower expert id, like a stable descending sort
        idx = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :topk]
    w = p.gather(1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-8) * scaling
    return idx.to(torch.int32), w


def moe_experts(x, idx, w, w13_packed, s13, w2_packed, s2, limit):
    """Routed experts, W4A16: per route  h = swiglu(bf16(x @ W13^T)) -> bf16;  y = bf16(h @ W2^T) * bf16(w);
    routes of a token are summed in fp32 and returned as bf16.  w13 [E, 2I, H/2] packed (gate rows first),
    w2 [E, H, I/2]  (python/minisgl/kernel/marlin_wna16.py:288-356)."""
    t, hdim = x.shape
    out = torch.zeros(t, hdim, dtype=torch.float32, device=x.device)
    for e in idx.unique().tolist():
        if e < 0:
            continue
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        w13 = quant.fp4_dequant(w13_packed[e], s13[e], dtype=torch.float32)
        w2 = quant.fp4_dequant(w2_packed[e], s2[e], dtype=torch.float32)
        g = (x[tok].float() @ w13.t()).to(torch.bfloat16)
        a = silu_mul_clamp(g, limit)
        y = (a.float() @ w2.t()).to(torch.bfloat16)
        y = (y * w[tok, slot].to(torch.bfloat16)[:, None]).float()
        out.index_add_(0, tok, y)
    return out.to(torch.bfloat16)


# --------------------------------------------------------------------------- sampling
def sample(logits, temperature, top_k, top_p, uniform):
    """Greedy where temperature <= 0, else inverse-CDF sampling with the given uniform numbers after
    top-k / top-p filtering of softmax(logits / T).  All per-row tensors; returns int64 [B]."""
    b, v = logits.shape
    greedy = logits.argmax(-1)
    out = greedy.clone()
    for r in range(b):
        tmp = float(temperature[r])
        if tmp <= 0 or int(top_k[r]) == 1:
            continue
        p = torch.softmax(logits[r].float() / tmp, dim=-1)
        order = torch.sort(p, descending=True, stable=True)
        probs, ids = order.values, order.indices
        keep = torch.ones(v, dtype=torch.bool, device=logits.device)
        k = int(top_k[r])
        if k > 0:
            keep[k:] = False
        cum = probs.cumsum(0)
        tp = float(top_p[r])
        if tp < 1.0:
            keep &= (cum - probs) < tp
        probs = torch.where(keep, probs, torch.zeros_like(probs))
        cdf = probs.cumsum(0)
        u = float(uniform[r]) * float(cdf[-1])
        pick = int(torch.searchsorted(cdf, torch.tensor(u, device=cdf.device), right=True).clamp(max=v - 1))
        out[r] = ids[pick]
    return out


def topk_select(logits, lens, k: int):  # noqa: F811  (final definition: index-ordered output)
    """Per row: the k entries of logits[:len] that come first under (score desc, index asc), returned sorted by
    index; rows with len <= k keep 0..len-1; a non-finite score inside the valid range invalidates the row
    (len -1).  Returns (idx int32 [T,k] padded with -1, out_len int32 [T])  (csrc/jit/dsv4_topk_v1.cu:275-479;
    the reference emits score order, attention does not depend on it)."""
    t = logits.shape[0]
    idx = torch.full((t, k), -1, dtype=torch.int32, device=logits.device)
    out_len = torch.zeros(t, dtype=torch.int32, device=logits.device)
    for r in range(t):
        n = min(int(lens[r]), logits.shape[1])
        if n <= 0:
            continue
        if n <= k:
            idx[r, :n] = torch.arange(n, dtype=torch.int32, device=logits.device)
            out_len[r] = n
            continue
        row = logits[r, :n].float()
        if not bool(torch.isfinite(row).all()):
            out_len[r] = -1
            continue
        vals = row.tolist()
        order = sorted(sorted(range(n), key=lambda i: (-vals[i], i))[:k])
        idx[r] = torch.tensor(order, dtype=torch.int32, device=logits.device)
        out_len[r] = k
    return idx, out_len


def sample(logits, temperature, top_k, top_p, uniform, mask_ids=None):  # noqa: F811
    """Greedy where temperature <= 0 or top_k == 1.  Otherwise p = softmax(logits / T); with the vocabulary ordered
    by (p desc, id asc) rank r is kept iff (top_k <= 0 or r < top_k) and the mass before it is < top_p; the sample
    is the first kept id, in id order, whose running kept mass exceeds u * kept_mass.  ``mask_ids`` [B, n] are ids
    forced to -inf first.  Returns int64 [B]."""
    b, v = logits.shape
    lg = logits.double().clone()
    if mask_ids is not None:
        for r in range(b):
            lg[r, mask_ids[r].long()] = float("-inf")
    out = lg.argmax(-1)
    for r in range(b):
        tmp = float(temperature[r])
        k = int(top_k[r])
        if tmp <= 0 or k == 1:
            continue
        p = torch.softmax(lg[r] / tmp, dim=-1)
        order = torch.sort(p, descending=True, stable=True).indices
        ps = p[order]
        before = ps.cumsum(0) - ps
        keep_sorted = before < float(top_p[r]) if float(top_p[r]) < 1.0 else torch.ones(v, dtype=torch.bool)
        if k > 0:
            keep_sorted = keep_sorted & (torch.arange(v) < k)
        keep = torch.zeros(v, dtype=torch.bool)
        keep[order[keep_sorted]] = True
        pk = torch.where(keep, p, torch.zeros_like(p))
        cdf = pk.cumsum(0)
        target = float(uniform[r]) * float(cdf[-1])
        pick = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True).clamp(max=v - 1))
        out[r] = pick
    return out
