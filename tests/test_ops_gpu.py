"""Each sm_100a kernel against the fp32 PyTorch oracle (minisgl.ops.ref) of the same operator, at the flagship
per-layer shapes (hidden 4096, head dim 512, rope 64, indexer 64 x 128)."""
import math
import types

import pytest
import torch

from minisgl.ops import api as O
from minisgl.ops import quant, ref
from minisgl.ops.ref import RopeSpec

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROPE = RopeSpec.make(64, 160000.0, 65536, 16.0, 32, 1)
ROPE0 = RopeSpec.make(64, 10000.0)


def bf(*shape, std=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)


def close(a, b, atol=2e-2, rtol=2e-2, frac=1.0):
    a, b = a.float().cpu(), b.float().cpu()
    ok = (a - b).abs() <= atol + rtol * b.abs()
    assert ok.float().mean().item() >= frac, ((a - b).abs().max().item(), ok.float().mean().item())


def test_embed_rmsnorm_silu_addcast():
    w = bf(1000, 4096)
    ids = torch.randint(0, 1000, (37,), dtype=torch.int32)
    out = O.embed(ids.to(DEV), w.to(DEV), 4)
    assert torch.equal(out.cpu(), w[ids.long()].unsqueeze(1).repeat(1, 4, 1))
    x, g = bf(37, 1536, seed=1), bf(1024, std=0.3, seed=2) + 1
    close(O.rms_norm(x.to(DEV)[:, :1024], g.to(DEV), 1e-6), ref.rms_norm(x[:, :1024], g, 1e-6))
    gu = bf(19, 4096, std=3.0, seed=3)
    close(O.silu_mul_clamp(gu.to(DEV), 7.0), ref.silu_mul_clamp(gu, 7.0))
    a, b = bf(9, 4096, seed=4), bf(9, 4096, seed=5)
    nvalid = torch.tensor([7], dtype=torch.int32, device=DEV)
    o = O.add_cast(a.to(DEV), b.to(DEV), nvalid).cpu()
    exp = (a.float() + b.float()).to(torch.bfloat16)
    exp[7:] = 0
    assert torch.equal(o, exp)


def test_embed_token_feedback_and_greedy_tail():
    """Decode rows take their token from the device-resident feedback buffer (embedding kernel gathers it and fills
    the id buffer); the greedy tail is an argmax with lowest-index ties that also scatters the token back."""
    w = bf(500, 4096, seed=40)
    feedback = torch.randint(0, 500, (9,), dtype=torch.int32)
    slots = torch.tensor([3, 0, 8, 8, 5], dtype=torch.int32)
    ids = torch.full((5,), -1, dtype=torch.int32, device=DEV)
    out = O.embed(ids, w.to(DEV), 4, feedback.to(DEV), slots.to(DEV))
    want = feedback[slots.long()]
    assert torch.equal(ids.cpu(), want) and torch.equal(out.cpu(), w[want.long()].unsqueeze(1).repeat(1, 4, 1))
    g = torch.Generator().manual_seed(41)
    logits = torch.randn(6, 129280 // 8, generator=g)
    logits[2, 77] = logits[2, 4000] = 50.0                        # a tie: the lower index wins
    logits[4] = float("-inf")
    fb_dev = torch.full((9,), -7, dtype=torch.int32, device=DEV)
    sl = torch.tensor([1, 2, 3, 4, 5, 6], dtype=torch.int32, device=DEV)
    nvalid = torch.tensor([5], dtype=torch.int32, device=DEV)
    toks = O.greedy_tokens(logits.to(DEV), 1000, sl, nvalid, fb_dev)
    exp = logits.argmax(-1) + 1000
    exp[2], exp[4] = 1077, 1000                                     # all -inf: the first column of the shard
    assert toks.cpu().tolist() == exp.tolist()
    assert fb_dev.cpu().tolist() == [-7] + exp[:5].tolist() + [-7, -7, -7]   # row 5 is padding: not fed back
    cpu_fb = torch.full((9,), -7, dtype=torch.int32)
    cpu = O.greedy_tokens(logits[:4], 1000, sl.cpu()[:4], None, cpu_fb)
    assert cpu.tolist() == exp[:4].tolist() and cpu_fb.tolist()[1:5] == exp[:4].tolist()


@pytest.mark.parametrize("block", [128, 64])
def test_fp8_quant_matches_oracle(block):
    x = bf(33, 1024, std=2.0, seed=6)
    x[0, :128] = 0
    q, s = O.fp8_quant(x.to(DEV), block)
    qr, sr = quant.fp8_act_quant(x, block)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8))


def test_rope_and_qkv_norm_store():
    t, h = 21, 8
    pos = torch.randint(0, 200000, (t,), dtype=torch.int32)
    x = bf(t, h, 512, seed=7)
    y = O.rope_tail(x.to(DEV).clone(), pos.to(DEV), ROPE, inverse=True)
    close(y, ref.rope_tail(x, pos, ROPE, True).to(torch.bfloat16), atol=3e-2)
    q, qkv, kw = bf(t, h, 512, seed=8), bf(t, 1536, seed=9), bf(512, std=0.2, seed=10) + 1
    ps = 256
    swa = torch.zeros(4 * ps, 512, dtype=torch.bfloat16)
    swa_map = torch.tensor([2, -1, 0, 3], dtype=torch.int32)
    out_loc = torch.randperm(3 * ps)[:t].to(torch.int32)
    out_loc[3] = -1
    qd, kvd = q.to(DEV), qkv.to(DEV)
    swad = swa.to(DEV)
    O.q_kv_norm_rope_store(qd, kvd[:, 1024:], pos.to(DEV), kw.to(DEV), 1e-6, ROPE, swad, out_loc.to(DEV),
                           swa_map.to(DEV), ps, True)
    qo, ko = O.q_kv_norm_rope_store(q.clone(), qkv[:, 1024:].clone(), pos, kw, 1e-6, ROPE, swa, out_loc, swa_map, ps,
                                    True)
    close(qd, qo, atol=3e-2)
    close(kvd[:, 1024:], ko, atol=3e-2, frac=0.995)  # an e4m3 rounding flip in the QAT moves one value by an fp8 ulp
    close(swad, swa, atol=3e-2, frac=0.999)
    assert torch.equal(kvd[:, :1024].cpu(), qkv[:, :1024])


def test_hc_pre_post_head():
    t, h = 11, 4096
    x = bf(t, 4, h, seed=11)
    fn, sc, base = bf(24, 4 * h, std=0.02, seed=12), torch.tensor([1.0, 0.7, 1.3]), torch.randn(24) * 0.5
    nw = bf(h, std=0.2, seed=13) + 1
    y, post, comb = O.hc_pre(x.to(DEV), fn.to(DEV), sc.to(DEV), base.to(DEV), 20, 1e-6, 1e-6, nw.to(DEV))
    yr, pr, cr = O.hc_pre(x, fn, sc, base, 20, 1e-6, 1e-6, nw)
    close(post, pr, atol=1e-3)
    close(comb, cr, atol=1e-3)
    close(y, yr, atol=3e-2)
    yy = bf(t, h, seed=14)
    close(O.hc_post(yy.to(DEV), x.to(DEV), post, comb), ref.hc_post(yy, x, pr, cr), atol=4e-2)
    fh = bf(4, 4 * h, std=0.02, seed=15)
    close(O.hc_head(x.to(DEV), fh.to(DEV), sc[:1].to(DEV), base[:4].to(DEV), 1e-6, 1e-6, nw.to(DEV)),
          O.hc_head(x, fh, sc[:1], base[:4], 1e-6, 1e-6, nw), atol=3e-2)


def _fb(pos, slots, page_table, out_loc=None, max_context=None):
    return types.SimpleNamespace(positions=pos, slots=slots, page_table=page_table, out_loc=out_loc,
                                 max_context=max_context or int(pos.max()) + 1, num_valid=None, is_prefill=False)


def _mk_batch(ps=256, seed=0):
    """Two requests: slot 0 continues at position 250 with 20 tokens (crosses a page), slot 2 is a fresh prefill."""
    g = torch.Generator().manual_seed(seed)
    pt = torch.zeros(4, 1024, dtype=torch.int32)
    pages = torch.randperm(12, generator=g).tolist()
    for s in range(4):
        for k in range(3):
            p = pages[s * 3 + k]
            pt[s, k * ps:(k + 1) * ps] = torch.arange(p * ps, (p + 1) * ps, dtype=torch.int32)
    pos = torch.cat([torch.arange(250, 270), torch.arange(0, 300)]).to(torch.int32)
    slots = torch.cat([torch.zeros(20), torch.full((300,), 2)]).to(torch.int32)
    out_loc = pt[slots.long(), pos.long()]
    return pos, slots, pt, out_loc


@pytest.mark.parametrize("ratio,d", [(4, 512), (4, 128), (128, 512)])
def test_compress_pool_and_state(ratio, d):
    ps = 256
    pos, slots, pt, out_loc = _mk_batch(ps)
    t = pos.shape[0]
    c = 2 if ratio == 4 else 1
    proj = torch.randn(t, 2 * c * d)
    ape = torch.randn(ratio, c * d) * 0.5
    ring_len = 8 if ratio == 4 else ratio
    ring = torch.randn(4 * ring_len, 2 * c * d)
    ckpt = torch.randn(13 * 4, 2 * d) if ratio == 4 else None
    fb = _fb(pos, slots, pt, out_loc)
    ring_d, ckpt_d = ring.to(DEV), (ckpt.to(DEV) if ckpt is not None else None)
    fbd = _fb(pos.to(DEV), slots.to(DEV), pt.to(DEV), out_loc.to(DEV))
    out = O.compress(proj.to(DEV), fbd, ratio, d, ape.to(DEV), ring_d, ckpt_d, ps)
    exp = O.compress(proj, fb, ratio, d, ape, ring, ckpt, ps)
    close(out, exp, atol=1e-4, rtol=1e-4)
    close(ring_d, ring, atol=1e-5)
    if ckpt is not None:
        close(ckpt_d, ckpt, atol=1e-6)


def test_compress_store_and_indexer_producers():
    ps = 256
    pos, slots, pt, out_loc = _mk_batch(ps)
    t = pos.shape[0]
    fb, fbd = _fb(pos, slots, pt, out_loc), _fb(pos.to(DEV), slots.to(DEV), pt.to(DEV), out_loc.to(DEV))
    for ratio in (4, 128):
        pooled = torch.randn(t, 512)
        nw = bf(512, std=0.2, seed=20) + 1
        rows = 13 * max(ps // ratio, 1)
        cache = torch.zeros(rows, 512, dtype=torch.bfloat16)
        cache_d = cache.to(DEV)
        O.compress_store(pooled.to(DEV), fbd, nw.to(DEV), 1e-6, ROPE, cache_d, ps, ratio)
        O.compress_store(pooled, fb, nw, 1e-6, ROPE, cache, ps, ratio)
        close(cache_d, cache, atol=3e-2)
    pooled = torch.randn(t, 128)
    nwf = torch.rand(128) + 0.5
    vals, scales = torch.zeros(13 * 64, 128, dtype=torch.uint8), torch.zeros(13 * 64)
    vd, sd = vals.to(DEV), scales.to(DEV)
    O.indexer_kv_store(pooled.to(DEV), fbd, nwf.to(DEV), 1e-6, ROPE, vd, sd, ps)
    O.indexer_kv_store(pooled, fb, nwf, 1e-6, ROPE, vals, scales, ps)
    assert torch.equal(sd.cpu(), scales)
    dq = lambda v, s: v.view(quant.FP8).float() * s[:, None]
    close(dq(vd.cpu(), sd.cpu()), dq(vals, scales), atol=2e-2, frac=0.995)
    q, w = bf(t, 64, 128, seed=21), bf(t, 64, seed=22)
    qc, wf = O.indexer_q_encode(q.to(DEV), w.to(DEV), pos.to(DEV), ROPE, 128 ** -0.5, 64 ** -0.5)
    qr, wr = O.indexer_q_encode(q, w, pos, ROPE, 128 ** -0.5, 64 ** -0.5)
    close(wf, wr, atol=1e-6, rtol=1e-3)
    assert (qc.cpu() == qr).float().mean() > 0.995


def test_indexer_logits_and_topk():
    ps = 256
    g = torch.Generator().manual_seed(3)
    pt = torch.zeros(2, 4096, dtype=torch.int32)
    pages = torch.randperm(16, generator=g).tolist()
    for k in range(16):
        pt[1, k * ps:(k + 1) * ps] = torch.arange(pages[k] * ps, (pages[k] + 1) * ps, dtype=torch.int32)
    pos = torch.tensor([4000, 2100, 2047, 700, 3], dtype=torch.int32)
    slots = torch.ones(5, dtype=torch.int32)
    t = 5
    qc = torch.randn(t, 64, 128, generator=g).to(quant.FP8).view(torch.uint8)
    wf = torch.randn(t, 64, generator=g)
    vals = torch.randn(16 * 64, 128, generator=g).to(quant.FP8).view(torch.uint8)
    scales = torch.rand(16 * 64, generator=g) + 0.5
    fb = _fb(pos, slots, pt, None, 4001)
    fbd = _fb(pos.to(DEV), slots.to(DEV), pt.to(DEV), None, 4001)
    idx, ln = O.indexer_select(qc.to(DEV), wf.to(DEV), vals.to(DEV), scales.to(DEV), fbd, ps, 512)
    idx_r, ln_r = O.indexer_select(qc, wf, vals, scales, fb, ps, 512)
    assert torch.equal(ln.cpu(), ln_r)
    for r in range(t):
        a, b = set(idx[r].cpu().tolist()), set(idx_r[r].tolist())
        assert len(a ^ b) <= 4, (r, len(a ^ b))  # fp32 summation order may swap near-ties at the threshold
    # determinism and the tie rule on exact inputs
    from minisgl.ops import cuda

    lg = torch.zeros(2, 2048)
    lg[0, 100:900] = 1.0
    lg[1] = torch.arange(2048).float()
    p2 = torch.tensor([8191, 8191], dtype=torch.int32)
    o1 = torch.empty(2, 512, dtype=torch.int32, device=DEV)
    l1 = torch.empty(2, dtype=torch.int32, device=DEV)
    cuda.nv.call("topk", cuda.nv.ptr(lg.to(DEV)), cuda.I(2048), cuda.nv.ptr(p2.to(DEV)), cuda.nv.ptr(o1),
                 cuda.nv.ptr(l1), cuda.I(2), cuda.I(512))
    assert o1[0].cpu().tolist() == list(range(100, 612))
    assert o1[1].cpu().tolist() == list(range(1536, 2048))


@pytest.mark.parametrize("prefill", [False, True])
def test_indexer_logits_tensor_core_kernel(prefill):
    """The tcgen05 logits kernel against the fp32 oracle and against the CUDA-core kernel: a prefill chunk whose
    rows run through two requests (groups of four rows share key tiles; one group straddles the request boundary)
    and a decode batch (every row its own request), ragged lengths, -inf past every row's length, and the row
    chunking that bounds the workspace."""
    from minisgl.ops import cuda

    ps = 256
    g = torch.Generator().manual_seed(11)
    pt = torch.zeros(4, 8192, dtype=torch.int32)
    pages = torch.randperm(64, generator=g).tolist()
    for s_ in range(2):
        for k in range(32):
            pg = pages[s_ * 32 + k]
            pt[s_ + 1, k * ps:(k + 1) * ps] = torch.arange(pg * ps, (pg + 1) * ps, dtype=torch.int32)
    if prefill:
        pos = torch.cat([torch.arange(5000, 5041), torch.arange(0, 30), torch.arange(8100, 8105)]).to(torch.int32)
        slots = torch.cat([torch.full((41,), 1), torch.full((30,), 2), torch.full((5,), 1)]).to(torch.int32)
    else:
        pos = torch.tensor([8191, 2, 3, 4095, 511, 512, 6000, 1023], dtype=torch.int32)
        slots = torch.tensor([1, 2, 1, 2, 1, 2, 1, 2], dtype=torch.int32)
    t = pos.shape[0]
    qc = (torch.randn(t, 64, 128, generator=g) * 2).to(quant.FP8).view(torch.uint8)
    wf = torch.randn(t, 64, generator=g)
    vals = (torch.randn(64 * 64, 128, generator=g) * 2).to(quant.FP8).view(torch.uint8)
    scales = torch.pow(2.0, torch.randint(-6, 3, (64 * 64,), generator=g).float())
    width = 2048
    a = [x.to(DEV) for x in (qc, wf, vals, scales, slots, pos, pt)]
    mma = cuda.indexer_logits(*a, ps, width, prefill).cpu()
    scalar = cuda.indexer_logits(*a, ps, width, prefill, force_scalar=True).cpu()
    j = torch.arange(width)
    n = ((pos.long() + 1) // 4).clamp(max=width)
    rows = (pt[slots.long()][:, (4 * j + 3).clamp(max=8191)].long() // ps) * 64 + ((4 * j + 3) % ps)[None, :] // 4
    want = ref.indexer_logits(qc, wf, vals, scales, rows, n)
    valid = j[None, :] < n[:, None]
    assert bool(torch.isinf(mma[~valid]).all()) and bool((mma[~valid] < 0).all())
    # e4m3 products are exact; only the order of the fp32 additions differs between the three
    scale = want[valid].abs().max()
    assert float((mma[valid] - want[valid]).abs().max()) <= 2e-4 * float(scale)
    assert float((mma[valid] - scalar[valid]).abs().max()) <= 2e-4 * float(scale)
    # selection through the public op, with the workspace bound forcing three row chunks
    fbd = _fb(a[5], a[4], a[6], None, 8192)
    fbd.is_prefill = prefill
    idx0, len0 = O.indexer_select(a[0], a[1], a[2], a[3], fbd, ps, 512)
    old = cuda.LOGITS_WORKSPACE_BYTES
    cuda.LOGITS_WORKSPACE_BYTES = width * 4 * max(t // 3, 1)
    try:
        idx1, len1 = O.indexer_select(a[0], a[1], a[2], a[3], fbd, ps, 512)
    finally:
        cuda.LOGITS_WORKSPACE_BYTES = old
    assert torch.equal(idx0, idx1) and torch.equal(len0, len1)
    fbc = _fb(pos, slots, pt, None, 8192)
    idx_r, len_r = O.indexer_select(qc, wf, vals, scales, fbc, ps, 512)
    assert torch.equal(len0.cpu(), len_r)
    for r in range(t):
        assert len(set(idx0[r].cpu().tolist()) ^ set(idx_r[r].tolist())) <= 4, r


@pytest.mark.parametrize("heads", [8, 64])
@pytest.mark.parametrize("ratio", [0, 4, 128])
def test_sparse_attention(heads, ratio):
    ps = 256
    g = torch.Generator().manual_seed(heads + ratio)
    pt = torch.zeros(3, 2048, dtype=torch.int32)
    pages = torch.randperm(8, generator=g).tolist()
    for k in range(8):
        pt[1, k * ps:(k + 1) * ps] = torch.arange(pages[k] * ps, (pages[k] + 1) * ps, dtype=torch.int32)
    pos = torch.tensor([0, 5, 127, 128, 1000, 2047], dtype=torch.int32)
    t = pos.shape[0]
    slots = torch.ones(t, dtype=torch.int32)
    swa_map = torch.randperm(9, generator=g).to(torch.int32)
    swa = bf(9 * ps, 512, seed=30)
    comp = bf(9 * max(ps // max(ratio, 1), 1), 512, seed=31) if ratio else None
    q = bf(t, heads, 512, seed=32)
    sink = torch.randn(heads, generator=g)
    tk_idx = tk_len = None
    if ratio == 4:
        tk_idx = torch.full((t, 512), -1, dtype=torch.int32)
        tk_len = torch.zeros(t, dtype=torch.int32)
        for r in range(t):
            n = min((int(pos[r]) + 1) // 4, 512)
            sel = torch.randperm(max((int(pos[r]) + 1) // 4, 1), generator=g)[:n].sort().values
            tk_idx[r, :n] = sel.to(torch.int32)
            tk_len[r] = n
    fb = _fb(pos, slots, pt, None, 2048)
    fbd = _fb(pos.to(DEV), slots.to(DEV), pt.to(DEV), None, 2048)
    dv = lambda x: None if x is None else x.to(DEV)
    o = O.attention(q.to(DEV), fbd, swa.to(DEV), swa_map.to(DEV), dv(comp), ratio, dv(tk_idx), dv(tk_len),
                    sink.to(DEV), 512 ** -0.5, ps, 128)
    o_r = O.attention(q, fb, swa, swa_map, comp, ratio, tk_idx, tk_len, sink, 512 ** -0.5, ps, 128)
    close(o, o_r, atol=2e-2)
    # inverse RoPE of the output tail fused into the epilogue == attention followed by rope_tail(inverse)
    spec = RopeSpec.make(64, 10000.0, 65536, 16.0, 32, 1)
    o2 = O.attention(q.to(DEV), fbd, swa.to(DEV), swa_map.to(DEV), dv(comp), ratio, dv(tk_idx), dv(tk_len),
                     sink.to(DEV), 512 ** -0.5, ps, 128, out_rope=spec)
    o2_r = O.rope_tail(o.clone(), fbd.positions, spec, inverse=True)
    assert torch.equal(o2[..., :448], o[..., :448])
    close(o2, o2_r, atol=1e-2)
    # split-KV: the token's key tiles spread over several CTAs and merged must give the one-CTA result (same
    # arithmetic up to the order of the fp32 additions), for split counts that leave some CTAs without any key too
    from minisgl.ops import cuda

    one = cuda.attention(q.to(DEV), fbd, swa.to(DEV), swa_map.to(DEV), dv(comp), ratio, dv(tk_idx), dv(tk_len),
                         sink.to(DEV), 512 ** -0.5, ps, 128, out_rope=spec, nsplit=1)
    close(one, O.rope_tail(o_r.to(DEV), fbd.positions, spec, inverse=True), atol=2e-2)
    for ns in (2, 5, 32):
        many = cuda.attention(q.to(DEV), fbd, swa.to(DEV), swa_map.to(DEV), dv(comp), ratio, dv(tk_idx), dv(tk_len),
                              sink.to(DEV), 512 ** -0.5, ps, 128, out_rope=spec, nsplit=ns)
        close(many, one, atol=4e-3, rtol=1e-2)
        again = cuda.attention(q.to(DEV), fbd, swa.to(DEV), swa_map.to(DEV), dv(comp), ratio, dv(tk_idx),
                               dv(tk_len), sink.to(DEV), 512 ** -0.5, ps, 128, out_rope=spec, nsplit=ns)
        assert torch.equal(many, again)          # the merge runs in split order whichever CTA finishes last


def test_moe_gate_and_experts():
    g = torch.Generator().manual_seed(5)
    t, h, e, inter, k = 45, 4096, 16, 512, 6
    y = bf(t, h, seed=40)
    gw = bf(e, h, std=0.1, seed=41).float()
    bias = torch.randn(e, generator=g) * 0.01
    ids = torch.randint(0, 100, (t,), dtype=torch.int32)
    idx, wt = O.moe_gate(y.to(DEV), gw.to(DEV), bias.to(DEV), k, 1.5, "sqrtsoftplus", None, ids.to(DEV))
    idx_r, wt_r = O.moe_gate(y, gw, bias, k, 1.5, "sqrtsoftplus", None, ids)
    same = (idx.cpu().sort(-1).values == idx_r.sort(-1).values).all(-1).float().mean()
    assert same > 0.9, same
    w13, s13 = quant.fp4_quant(torch.randn(e, 2 * inter, h, generator=g) * 0.02)
    w2, s2 = quant.fp4_quant(torch.randn(e, h, inter, generator=g) * 0.02)
    out = O.moe_experts(y.to(DEV), idx_r.to(DEV), wt_r.to(DEV), w13.to(DEV), s13.to(DEV), w2.to(DEV), s2.to(DEV),
                        7.0, 0)
    exp = O.moe_experts(y, idx_r, wt_r, w13, s13, w2, s2, 7.0, 0)
    close(out, exp, atol=3e-2, rtol=3e-2, frac=0.999)
    # expert-parallel slice: only experts [8, 16) are local
    out2 = O.moe_experts(y.to(DEV), idx_r.to(DEV), wt_r.to(DEV), w13[8:].to(DEV), s13[8:].to(DEV), w2[8:].to(DEV),
                         s2[8:].to(DEV), 7.0, 8)
    exp2 = O.moe_experts(y, idx_r, wt_r, w13[8:], s13[8:], w2[8:], s2[8:], 7.0, 8)
    close(out2, exp2, atol=3e-2, rtol=3e-2, frac=0.999)


def test_moe_experts_many_routes_per_expert():
    g = torch.Generator().manual_seed(6)
    t, h, e, inter, k = 700, 4096, 4, 256, 2
    y = bf(t, h, seed=42)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32)
    wt = torch.rand(t, k, generator=g)
    w13, s13 = quant.fp4_quant(torch.randn(e, 2 * inter, h, generator=g) * 0.02)
    w2, s2 = quant.fp4_quant(torch.randn(e, h, inter, generator=g) * 0.02)
    out = O.moe_experts(y.to(DEV), idx.to(DEV), wt.to(DEV), w13.to(DEV), s13.to(DEV), w2.to(DEV), s2.to(DEV), 7.0, 0)
    exp = O.moe_experts(y, idx, wt, w13, s13, w2, s2, 7.0, 0)
    close(out, exp, atol=3e-2, rtol=3e-2, frac=0.999)


@pytest.mark.parametrize("e_local,m", [(32, 128), (16, 1024)])
def test_moe_full_size_repeatable(e_local, m):
    """Full-size expert shapes, many work items per CTA, partly filled route tiles: repeated calls must agree bit for
    bit (the route order inside an expert changes from call to call, the result may not) and match the oracle."""
    h, inter, topk = 4096, 2048, 6
    g = torch.Generator().manual_seed(11)
    w13 = torch.randint(0, 256, (e_local, 2 * inter, h // 2), generator=g, dtype=torch.uint8).view(torch.int8)
    s13 = torch.randint(119, 122, (e_local, 2 * inter, h // 32), generator=g, dtype=torch.uint8)
    w2 = torch.randint(0, 256, (e_local, h, inter // 2), generator=g, dtype=torch.uint8).view(torch.int8)
    s2 = torch.randint(119, 122, (e_local, h, inter // 32), generator=g, dtype=torch.uint8)
    y = bf(m, h, seed=3)
    idx = torch.stack([torch.randperm(256, generator=g)[:topk] for _ in range(m)]).to(torch.int32)
    wt = torch.rand(m, topk, generator=g)
    dev = [a.to(DEV) for a in (y, idx, wt, w13, s13, w2, s2)]
    outs = [O.moe_experts(*dev, 7.0, 0) for _ in range(8)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    exp = O.moe_experts(y, idx, wt, w13, s13, w2, s2, 7.0, 0).float()
    got = outs[0].float().cpu()
    assert float((got - exp).norm() / exp.norm()) < 2e-3
    close(got, exp, atol=0.13, rtol=3e-2)


def test_moe_mx_split_is_exact_for_bf16():
    """The block-scaled expert kernel writes every bf16 activation as hi + lo (two e4m3 values under one power-of-two
    scale per 32 elements each).  For every element within 2^13 of its block's largest magnitude the pair must give the
    bf16 value back bit for bit; smaller ones may be off by at most 2^-21 of that magnitude."""
    from minisgl.ops import cuda as C
    from minisgl.ops import native as nv
    from minisgl.ops.native import I

    t, h, e, k, nt = 45, 4096, 16, 6, 8
    g = torch.Generator().manual_seed(1)
    y = (torch.randn(t, h, generator=g) * torch.exp(torch.randn(t, h, generator=g) * 2)).to(torch.bfloat16).to(DEV)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32).to(DEV)
    wt = torch.rand(t, k, generator=g).to(DEV)
    routes = t * k
    max_tiles = min(e, routes) + routes // nt + 1
    plan = torch.empty(4 + 3 * max_tiles + 3 * routes, dtype=torch.int32, device=DEV)
    nv.call("moe_plan", nv.ptr(idx), nv.ptr(wt), I(routes), I(e), I(0), I(nt), nv.ptr(plan), I(max_tiles))
    xq = torch.zeros(2 * routes, h, dtype=torch.uint8, device=DEV)
    sfx = torch.zeros(max_tiles, h // 128, 512, dtype=torch.uint8, device=DEV)
    nv.call("moe_mx_permute", nv.ptr(y), nv.ptr(xq), nv.ptr(sfx), nv.ptr(plan), I(routes), I(max_tiles), I(k), I(h),
            I(nt))
    torch.cuda.synchronize()
    p = plan.cpu()
    ntiles = int(p[0])
    tiles = p[4:4 + 3 * max_tiles].view(max_tiles, 3)
    sroute = p[4 + 3 * max_tiles: 4 + 3 * max_tiles + routes]
    xqc, sfc, yc = xq.cpu(), sfx.cpu(), y.cpu().float()
    blk = torch.arange(h) // 32
    seen = 0
    for ti in range(ntiles):
        _, tok0, ntok = [int(v) for v in tiles[ti]]
        assert 1 <= ntok <= nt
        for n in range(ntok):
            pos = tok0 + n
            x = yc[int(sroute[pos]) // k]
            hi = xqc[2 * pos].view(torch.float8_e4m3fn).float()
            lo = xqc[2 * pos + 1].view(torch.float8_e4m3fn).float()
            off = lambda row: (row % 32) * 16 + (row // 32) * 4 + (blk % 4)
            eh = sfc[ti, blk // 4, off(2 * n)].float()
            el = sfc[ti, blk // 4, off(2 * n + 1)].float()
            rec = hi * torch.exp2(eh - 127) + lo * torch.exp2(el - 127)
            bmax = x.abs().view(-1, 32).max(-1).values.repeat_interleave(32)
            big = x.abs() >= bmax * 2.0 ** -13
            assert torch.equal(rec[big], x[big])
            assert bool(((rec - x).abs() <= bmax * 2.0 ** -21).all())
            seen += 1
    assert seen == routes  # every expert is resident: every route has a position


def _flush_l2():
    if not hasattr(_flush_l2, "buf"):
        _flush_l2.buf = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    _flush_l2.buf.zero_()


@pytest.mark.parametrize("m,expect_nt", [(128, 8), (256, 16), (600, 32), (2048, 64)])
def test_moe_mx_every_tile_width_cold_and_warm(m, expect_nt):
    """One rank of an 8-way expert-parallel layer (32 of 256 experts resident), full-size experts: the block-scaled
    kernel at each route-tile width against the fp16-operand kernel (both compute the exact bf16 x FP4 products with
    fp32 accumulation; they differ in summation order only), bit-identical from call to call, also when every call
    starts from a flushed L2 (weights, plan and route rows then arrive from HBM and every pipeline wait is taken)."""
    from minisgl.ops import cuda as C

    h, inter, topk, e_local = 4096, 2048, 6, 32
    assert C.route_tile(m * topk, 256, "mx") == expect_nt
    g = torch.Generator().manual_seed(11)
    w13 = torch.randint(0, 256, (e_local, 2 * inter, h // 2), generator=g, dtype=torch.uint8).view(torch.int8)
    s13 = torch.randint(119, 122, (e_local, 2 * inter, h // 32), generator=g, dtype=torch.uint8)
    w2 = torch.randint(0, 256, (e_local, h, inter // 2), generator=g, dtype=torch.uint8).view(torch.int8)
    s2 = torch.randint(119, 122, (e_local, h, inter // 32), generator=g, dtype=torch.uint8)
    y = bf(m, h, seed=3)
    idx = torch.stack([torch.randperm(256, generator=g)[:topk] for _ in range(m)]).to(torch.int32)
    wt = torch.rand(m, topk, generator=g)
    dev = [a.to(DEV) for a in (y, idx, wt, w13, s13, w2, s2)]

    def run():
        rows, plan, mt = C.moe_routed(*dev, 7.0, 0, 256)
        return C.moe_finalize(rows, plan, mt, None, None, m, topk, h)

    assert C.MOE_KERNEL == "mx"
    C.MOE_KERNEL = "f16"
    try:
        want = run().float()
    finally:
        C.MOE_KERNEL = "mx"
    first = run()
    assert float((first.float() - want).norm() / want.norm()) < 1e-3
    for i in range(5):
        if i >= 2:
            _flush_l2()
        assert torch.equal(run(), first), f"call {i} differs"


def test_fused_quant_matches_separate_quant():
    """The producers that also write FP8 (rms_norm, hc_pre, SwiGLU) give exactly what fp8_quant gives on their
    bf16 result."""
    from minisgl.ops import cuda as C

    g = torch.Generator().manual_seed(21)
    x = (torch.randn(40, 1024, generator=g) * 3).to(torch.bfloat16).to(DEV)
    w = torch.rand(1024, generator=g).to(torch.bfloat16).to(DEV)
    y, (q, s) = O.rms_norm(x, w, 1e-6, want_q=True)
    q2, s2 = O.fp8_quant(y)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)

    gu = (torch.randn(33, 2 * 512, generator=g) * 4).to(torch.bfloat16).to(DEV)
    qa, sa = O.silu_mul_clamp_quant(gu, 7.0)
    qb, sb = O.fp8_quant(O.silu_mul_clamp(gu, 7.0))
    assert torch.equal(qa.view(torch.uint8), qb.view(torch.uint8)) and torch.equal(sa, sb)

    t, h = 24, 1024
    xs = (torch.randn(t, 4, h, generator=g)).to(torch.bfloat16).to(DEV)
    fn = (torch.randn(24, 4 * h, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    scale = torch.rand(3, generator=g).to(DEV)
    base = torch.randn(24, generator=g).to(DEV) * 0.1
    nw = torch.rand(h, generator=g).to(torch.bfloat16).to(DEV)
    yy, post, comb, (qh, sh) = O.hc_pre(xs, fn, scale, base, 20, 1e-6, 1e-6, nw, want_q=True)
    q3, s3 = O.fp8_quant(yy)
    assert torch.equal(qh.view(torch.uint8), q3.view(torch.uint8)) and torch.equal(sh, s3)
    y0, p0, c0 = O.hc_pre(xs, fn, scale, base, 20, 1e-6, 1e-6, nw)
    assert torch.equal(y0, yy) and torch.equal(p0, post) and torch.equal(c0, comb)


def test_sampling():
    g = torch.Generator().manual_seed(7)
    b, v = 6, 129280
    lg = torch.randn(b, v, generator=g) * 3
    temp = torch.tensor([0.0, 1.0, 0.7, 1.0, 1.3, 0.5])
    tk = torch.tensor([-1, 1, -1, 40, 5, -1], dtype=torch.int32)
    tp = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.9, 0.8])
    u = torch.rand(b, generator=g)
    mask = torch.stack([lg.argmax(-1), torch.zeros(b, dtype=torch.long)], 1).to(torch.int32)
    out = O.sample(lg.to(DEV), temp.to(DEV), tk.to(DEV), tp.to(DEV), u.to(DEV), mask.to(DEV))
    exp = O.sample(lg, temp, tk, tp, u, mask)
    assert torch.equal(out.cpu(), exp), (out.cpu(), exp)
    assert torch.equal(O.argmax(lg.to(DEV)).cpu(), lg.argmax(-1))


@pytest.mark.gpu
def test_index_audit_records_a_violation_without_touching_memory():
    """The checked-run audit kernel: in-range indices leave the status word clear; an out-of-range entry is recorded
    as code 2 with the caller's tag and the entry's position, nothing is dereferenced, and kernels still run after."""
    from minisgl.ops import api as O
    from minisgl.ops import native

    native.read_status(clear=True)
    idx = torch.randint(0, 1000, (5000,), device="cuda", dtype=torch.int32)
    idx[17] = -1
    O.check_index(idx, -1, 1000, "out_loc")
    assert native.read_status()[0] == 0
    idx[4321] = 1000
    O.check_index(idx, -1, 1000, "out_loc")
    st = native.read_status(clear=True)
    assert st[0] == 2 and st[1] == O.INDEX_TAGS["out_loc"] and st[2] == 4321, st
    O.check_index(idx[:4000].contiguous(), -1, 1000, "out_loc")
    assert native.read_status()[0] == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
