"""Operator microbenchmarks at the model's shapes (the reference ships ~27 such scripts: quantised linear, wo_a,
router, hyper-connections, norms, SwiGLU, sampling ...).  One registry, one timing method: every operator is captured
`calls` times in a CUDA graph (launch overhead amortised, as in the engine) and the per-call time is reported with the
bytes it must move and the fraction of the measured HBM copy bandwidth that this corresponds to.  Working sets are
rotated over several weight copies so that the weights do not stay in L2 between calls.

    python -m minisgl.benchmark.ops --tp 8 --rows 128            # all operators
    python -m minisgl.benchmark.ops --only wq_b router hc_pre

The attention / indexer / top-k / compressor kernels run on a synthetic paged cache (random rows, shuffled pages):
with ``--prefill 0`` every row is a decode token of its own request at position ``--context - 1``, with ``--prefill 1``
the rows are one request's chunk that ends at ``--context``.  The FP4 expert GEMM has its own script
(``minisgl.benchmark.moe_gemm``), whole steps ``minisgl.benchmark.decode_step``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _hbm():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        return json.load(open(path))["hbm_gbs"], "measured"
    except Exception:
        return 6650.0, "fallback"


def build_cache_ops(tp: int, rows: int, ctx: int, prefill: bool, dev, ops: dict) -> None:
    """Attention (window / 4:1 selected / 128:1), indexer logits (tensor-core and CUDA-core kernels), top-k, the
    compressor pooling + state kernels and the indexer's producers, on a synthetic cache."""
    import types

    from minisgl.ops import api as O
    from minisgl.ops import cuda as C
    from minisgl.ops import quant
    from minisgl.ops.ref import RopeSpec

    ps, D, DI, HI, K = 256, 512, 128, 64, 512
    hl = 64 // tp
    g = torch.Generator(device=dev).manual_seed(1)
    nreq = 1 if prefill else rows
    ppr = (ctx + ps - 1) // ps                      # pages per request
    npages = nreq * ppr
    perm = torch.randperm(npages, device=dev, generator=g).to(torch.int32)
    pt = torch.zeros(nreq + 1, ppr * ps, dtype=torch.int32, device=dev)
    ar = torch.arange(ps, dtype=torch.int32, device=dev)
    for r in range(nreq):
        pt[r] = (perm[r * ppr:(r + 1) * ppr, None] * ps + ar[None, :]).reshape(-1)
    if prefill:
        pos = torch.arange(ctx - rows, ctx, dtype=torch.int32, device=dev)
        slots = torch.zeros(rows, dtype=torch.int32, device=dev)
    else:
        pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
        slots = torch.arange(rows, dtype=torch.int32, device=dev)
    out_loc = pt[slots.long(), pos.long()].contiguous()
    fb = types.SimpleNamespace(positions=pos, slots=slots, page_table=pt, out_loc=out_loc, max_context=ctx,
                               num_valid=None, is_prefill=prefill)
    swa = (torch.randn(npages * ps, D, device=dev, generator=g)).to(torch.bfloat16)
    swa_map = torch.arange(npages + 1, dtype=torch.int32, device=dev)
    c4 = torch.randn(npages * (ps // 4), D, device=dev, generator=g).to(torch.bfloat16)
    c128 = torch.randn(npages * (ps // 128), D, device=dev, generator=g).to(torch.bfloat16)
    q = torch.randn(rows, hl, D, device=dev, generator=g).to(torch.bfloat16)
    sink = torch.randn(hl, device=dev, generator=g)
    rope = RopeSpec.make(64, 160000.0, 65536, 16.0, 32, 1)
    n4 = (pos.long() + 1) // 4
    sel = torch.full((rows, K), -1, dtype=torch.int32, device=dev)
    sel_len = torch.minimum(n4, torch.tensor(K, device=dev)).to(torch.int32)
    for r in range(rows):
        n = int(n4[r])
        k = min(n, K)
        sel[r, :k] = torch.randperm(max(n, 1), device=dev, generator=g)[:k].sort().values.to(torch.int32)
    win = min(ctx, 128)
    row_bytes = D * 2
    ops["attn_window"] = (lambda: O.attention(q, fb, swa, swa_map, None, 0, None, None, sink, D ** -0.5, ps, 128,
                                              out_rope=rope), rows * (win + 2 * hl) * row_bytes)
    ops["attn_c4_selected"] = (lambda: O.attention(q, fb, swa, swa_map, c4, 4, sel, sel_len, sink, D ** -0.5, ps, 128,
                                                   out_rope=rope),
                               int(sel_len.sum()) * row_bytes + rows * (win + 2 * hl) * row_bytes)
    ops["attn_c128_all"] = (lambda: O.attention(q, fb, swa, swa_map, c128, 128, None, None, sink, D ** -0.5, ps, 128,
                                                out_rope=rope),
                            int(((pos.long() + 1) // 128).sum()) * row_bytes + rows * (win + 2 * hl) * row_bytes)
    qc = torch.randn(rows, HI, DI, device=dev, generator=g).to(quant.FP8).view(torch.uint8)
    wf = torch.randn(rows, HI, device=dev, generator=g)
    vals = torch.randn(npages * (ps // 4), DI, device=dev, generator=g).to(quant.FP8).view(torch.uint8)
    scales = torch.rand(npages * (ps // 4), device=dev, generator=g) + 0.5
    width = (ctx // 4 + 63) // 64 * 64
    if width > K:
        lg = torch.empty(rows, width, dtype=torch.float32, device=dev)
        key_bytes = (int(n4.max()) if prefill else int(n4.sum())) * (DI + 4)
        flops = 2.0 * float(n4.sum()) * HI * DI
        ops["indexer_logits_tcgen05"] = (lambda: C.indexer_logits(qc, wf, vals, scales, slots, pos, pt, ps, width,
                                                                  prefill, out=lg),
                                         key_bytes + rows * HI * DI + rows * width * 4, flops)
        ops["indexer_logits_cuda_cores"] = (lambda: C.indexer_logits(qc, wf, vals, scales, slots, pos, pt, ps, width,
                                                                     prefill, out=lg, force_scalar=True),
                                            key_bytes + rows * HI * DI + rows * width * 4, flops)
        C.indexer_logits(qc, wf, vals, scales, slots, pos, pt, ps, width, prefill, out=lg)
        idx = torch.empty(rows, K, dtype=torch.int32, device=dev)
        ln = torch.empty(rows, dtype=torch.int32, device=dev)
        ops["indexer_topk"] = (lambda: C.nv.call("topk", C.nv.ptr(lg), C.I(width), C.nv.ptr(pos), C.nv.ptr(idx),
                                                 C.nv.ptr(ln), C.I(rows), C.I(K)), rows * width * 4 + rows * K * 4)
    proj4 = torch.randn(rows, 4 * D, device=dev, generator=g)
    proj128 = torch.randn(rows, 2 * D, device=dev, generator=g)
    ape4 = torch.randn(4, 2 * D, device=dev, generator=g)
    ape128 = torch.randn(128, D, device=dev, generator=g)
    ring4 = torch.zeros((nreq + 1) * 8, 4 * D, device=dev)
    ring128 = torch.zeros((nreq + 1) * 128, 2 * D, device=dev)
    ckpt = torch.zeros((npages + 1) * 4, 2 * D, device=dev)
    nw = torch.ones(D, dtype=torch.bfloat16, device=dev)

    def comp(ratio):
        proj, ape, ring, ck, cache = (proj4, ape4, ring4, ckpt, c4) if ratio == 4 else (proj128, ape128, ring128, None, c128)
        pooled = O.compress(proj, fb, ratio, D, ape, ring, ck, ps)
        O.compress_store(pooled, fb, nw, 1e-6, rope, cache, ps, ratio)

    ops["compress_c4_pool+state+store"] = (lambda: comp(4), rows * 4 * D * 4 * 2)
    ops["compress_c128_pool+state+store"] = (lambda: comp(128), rows * 2 * D * 4 * 2)
    iq = torch.randn(rows, HI, DI, device=dev, generator=g).to(torch.bfloat16)
    iw = torch.randn(rows, HI, device=dev, generator=g).to(torch.bfloat16)
    ops["indexer_q_encode"] = (lambda: O.indexer_q_encode(iq, iw, pos, rope, DI ** -0.5, HI ** -0.5),
                               rows * HI * DI * 3)


def build(tp: int, rows: int, dev):
    """Returns {name: (callable, algorithmic bytes per call)}; weights exist in `copies` rotated versions."""
    from minisgl.ops import api as O
    from minisgl.ops import gemm, quant

    H, QL, HD, HEADS, OL, OG, INTER, E, V = 4096, 1024, 512, 64, 1024, 8, 2048, 256, 129280
    hl, gl = HEADS // tp, max(OG // tp, 1)
    copies = 6
    g = torch.Generator(device=dev).manual_seed(0)

    def bf(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(torch.bfloat16)

    def fp8w(n, k):
        ws = []
        for _ in range(copies):
            wq, sc = quant.fp8_weight_quant(torch.randn(n, k, device=dev, generator=g) * 0.02)
            ws.append((wq, quant.e8m0_decode(sc)))
        return ws

    x = bf(rows, H)
    xq = O.fp8_quant(x)
    ql = bf(rows, QL)
    qlq = O.fp8_quant(ql)
    ops = {}
    state = {"i": 0}

    def rot(ws):
        state["i"] += 1
        return ws[state["i"] % copies]

    def linear(name, n, k, inp):
        ws = fp8w(n, k)
        ops[name] = (lambda: O.gemm_fp8(inp[0], inp[1], *rot(ws)), n * k + rows * k + rows * n * 2)

    linear("wqkv_a", QL + HD, H, xq)
    linear("wq_b", hl * HD, QL, qlq)
    oq = O.fp8_quant(bf(rows, gl * OL))
    linear("wo_b", H, gl * OL, oq)
    linear("shared_gate_up", 2 * INTER // tp, H, xq)
    aq = O.fp8_quant(bf(rows, INTER // tp))
    linear("shared_down", H, INTER // tp, aq)
    woa = [bf(gl * OL, hl * HD // gl, scale=0.02) for _ in range(copies)]
    o = bf(rows, hl * HD)
    ops["wo_a_grouped"] = (lambda: O.gemm_bf16_grouped(o, rot(woa), gl), gl * OL * (hl * HD // gl) * 2 + rows * hl * HD * 2)
    gate = [bf(E, H, scale=0.02) for _ in range(copies)]
    ops["router_partials"] = (lambda: gemm.gemm_bf16_partials(x, rot(gate)), E * H * 2 + rows * H * 2)
    head = [bf(V // tp, H, scale=0.02) for _ in range(2)]
    ops["lm_head"] = (lambda: O.gemm_bf16(x, head[state["i"] % 2], out_dtype=torch.float32), (V // tp) * H * 2)
    res = bf(rows, 4, H)
    fn = [bf(24, 4 * H, scale=0.02) for _ in range(copies)]
    sc3, base = torch.rand(3, device=dev), torch.randn(24, device=dev) * 0.1
    nw = torch.rand(H, device=dev).to(torch.bfloat16)
    ops["hc_pre+norm+quant"] = (lambda: O.hc_pre(res, rot(fn), sc3, base, 20, 1e-6, 1e-6, nw, want_q=True),
                                rows * 4 * H * 2 * 2 + 24 * 4 * H * 2)
    y, post, comb = O.hc_pre(res, fn[0], sc3, base, 20, 1e-6, 1e-6, nw)
    ops["hc_post"] = (lambda: O.hc_post(y, res, post, comb), rows * 4 * H * 2 * 2 + rows * H * 2)
    ops["rms_norm+quant"] = (lambda: O.rms_norm(ql, nw[:QL], 1e-6, want_q=True), rows * QL * 3)
    ops["fp8_quant"] = (lambda: O.fp8_quant(x), rows * H * 3)
    gu = bf(rows, 2 * INTER // tp)
    ops["silu_mul_clamp_quant"] = (lambda: O.silu_mul_clamp_quant(gu, 7.0), rows * INTER // tp * 5)
    logits = torch.randn(rows, V, device=dev, generator=g)
    temp = torch.full((rows,), 0.7, device=dev)
    tk = torch.full((rows,), 40, dtype=torch.int32, device=dev)
    tp_ = torch.full((rows,), 0.9, device=dev)
    u = torch.rand(rows, device=dev, generator=g)
    ops["sample_topk_topp"] = (lambda: O.sample(logits, temp, tk, tp_, u), rows * V * 4)
    ops["argmax"] = (lambda: O.argmax(logits), rows * V * 4)
    return ops


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--rows", type=int, default=128)
    ap.add_argument("--calls", type=int, default=24)
    ap.add_argument("--only", nargs="*", default=[])
    ap.add_argument("--context", type=int, default=0, help="> 0: also the attention / indexer / compressor kernels")
    ap.add_argument("--prefill", type=int, default=0, help="1: the rows are one request's prefill chunk")
    ap.add_argument("--cache-ops-only", action="store_true")
    ap.add_argument("--eager", type=int, default=0,
                    help="> 0: run every operator this many times eagerly and report nothing (profiler captures)")
    a = ap.parse_args(argv)
    from minisgl.benchmark.perf import time_in_graph
    from minisgl.ops import native

    dev = torch.device("cuda")
    hbm, src = _hbm()
    ops = {} if a.cache_ops_only else build(a.tp, a.rows, dev)
    if a.context > 0:
        build_cache_ops(a.tp, a.rows, a.context, bool(a.prefill), dev, ops)
    out = []
    for name, spec in ops.items():
        if a.only and name not in a.only:
            continue
        fn, nbytes = spec[0], spec[1]
        if a.eager > 0:
            for _ in range(a.eager):
                fn()
            torch.cuda.synchronize()
            continue
        ms = time_in_graph(fn, calls=a.calls)
        us = ms * 1e3
        gbs = nbytes / us / 1e3
        row = {"op": name, "rows": a.rows, "tp": a.tp, "us": round(us, 2), "algorithmic_MB": round(nbytes / 1e6, 2),
               "GBs": round(gbs, 1), f"frac_of_{src}_hbm": round(gbs / hbm, 3)}
        if a.context > 0:
            row["context"], row["prefill"] = a.context, bool(a.prefill)
        if len(spec) > 2:
            row["TFLOPs"] = round(spec[2] / us / 1e6, 2)
        out.append(row)
        print(json.dumps(row), flush=True)
    native.assert_device_ok()
    return out


if __name__ == "__main__":
    main()
