"""Operator microbenchmarks at the model's shapes (the reference ships ~27 such scripts: quantised linear, wo_a,
router, hyper-connections, norms, SwiGLU, sampling ...).  One registry, one timing method: every operator is captured
`calls` times in a CUDA graph (launch overhead amortised, as in the engine) and the per-call time is reported with the
bytes it must move and the fraction of the measured HBM copy bandwidth that this corresponds to.  Working sets are
rotated over several weight copies so that the weights do not stay in L2 between calls.

    python -m minisgl.benchmark.ops --tp 8 --rows 128            # all operators
    python -m minisgl.benchmark.ops --only wq_b router hc_pre

The attention / indexer / compressor kernels need a populated KV cache and are timed inside a real step by
``python -m minisgl.benchmark.decode_step --profile 1``; the FP4 expert GEMM by ``minisgl.benchmark.moe_gemm``.
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
    a = ap.parse_args(argv)
    from minisgl.benchmark.perf import time_in_graph
    from minisgl.ops import native

    dev = torch.device("cuda")
    hbm, src = _hbm()
    ops = build(a.tp, a.rows, dev)
    out = []
    for name, (fn, nbytes) in ops.items():
        if a.only and name not in a.only:
            continue
        ms = time_in_graph(fn, calls=a.calls)
        us = ms * 1e3
        gbs = nbytes / us / 1e3
        row = {"op": name, "rows": a.rows, "tp": a.tp, "us": round(us, 2), "algorithmic_MB": round(nbytes / 1e6, 2),
               "GBs": round(gbs, 1), f"frac_of_{src}_hbm": round(gbs / hbm, 3)}
        out.append(row)
        print(json.dumps(row), flush=True)
    native.assert_device_ok()
    return out


if __name__ == "__main__":
    main()
