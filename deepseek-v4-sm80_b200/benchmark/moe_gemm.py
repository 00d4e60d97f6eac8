"""Microbenchmark of the routed-expert path (plan, permute / split, FP4 grouped GEMM 1 and 2) with uniform-random routing.

    python -m minisgl.benchmark.moe_gemm --experts 32 --rows 128 [--iters 5]

Every timed call starts from a flushed L2.  The roofline of one grouped GEMM is the packed FP4 bytes plus scale bytes
of the experts that at least one route touches, divided by the measured HBM copy bandwidth.  ``--experts`` is the
number of experts resident on this GPU (256 = the whole layer, 32 = one rank of an 8-way expert-parallel layer); routes
that pick a non-resident expert are dropped, as expert parallelism does.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _hbm_gbs():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        return json.load(open(path))["hbm_gbs"], "measured"
    except Exception:
        return 6650.0, "fallback"


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--rows", type=int, default=128)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=6)
    a = ap.parse_args(argv)
    from minisgl.benchmark.perf import flush_l2
    from minisgl.ops import cuda as C
    from minisgl.ops import native

    dev, H, inter, topk, e_local, m = "cuda", a.hidden, a.inter, a.topk, a.experts, a.rows
    u8 = dict(device=dev, dtype=torch.uint8)
    w13 = torch.randint(0, 256, (e_local, 2 * inter, H // 2), **u8).view(torch.int8)
    s13 = torch.randint(119, 122, (e_local, 2 * inter, H // 32), **u8)
    w2 = torch.randint(0, 256, (e_local, H, inter // 2), **u8).view(torch.int8)
    s2 = torch.randint(119, 122, (e_local, H, inter // 32), **u8)
    x = torch.randn(m, H, device=dev).to(torch.bfloat16)
    gi = torch.Generator(device=dev).manual_seed(1234)
    idx = torch.stack([torch.randperm(256, device=dev, generator=gi)[:topk] for _ in range(m)]).to(torch.int32)
    idx = idx.contiguous()
    wt = torch.rand(m, topk, device=dev)
    touched = int(torch.unique(idx[idx < e_local]).numel())
    for _ in range(2):
        C.moe_routed(x, idx, wt, w13, s13, w2, s2, 7.0, 0, 256)
    torch.cuda.synchronize()
    native.enable_profile(True)
    for _ in range(a.iters):
        flush_l2()
        C.moe_routed(x, idx, wt, w13, s13, w2, s2, 7.0, 0, 256)
    # events in launch order: plan, permute, gemm(1), gemm(2)
    # (MINISGL_MOE_KERNEL=f16: moe_permute / moe_gemm; default: moe_mx_permute / moe_mx_gemm)
    ev = {"moe_plan": [], "moe_permute": [], "moe_gemm1": [], "moe_gemm2": []}
    seen = 0
    from minisgl.ops.native import _PROFILE  # per-launch events, in order

    torch.cuda.synchronize()
    for name, e0, e1 in _PROFILE["events"]:
        name = name.replace("moe_mx_", "moe_")
        if name == "moe_gemm":
            seen += 1
            name = "moe_gemm1" if seen % 2 == 1 else "moe_gemm2"
        ev.setdefault(name, []).append(e0.elapsed_time(e1) * 1e3)
    native.enable_profile(False)
    hbm, src = _hbm_gbs()
    us = {k: sorted(v)[len(v) // 2] for k, v in ev.items() if v}
    b1 = touched * (2 * inter * H // 2 + 2 * inter * H // 32)
    b2 = touched * (H * inter // 2 + H * inter // 32)
    out = {"kernel": C.MOE_KERNEL, "experts_resident": e_local, "experts_touched": touched, "rows": m, "median_us": us,
           "gemm1_gbs": b1 / us["moe_gemm1"] / 1e3, "gemm2_gbs": b2 / us["moe_gemm2"] / 1e3,
           "gemm1_frac_of_%s_hbm" % src: b1 / us["moe_gemm1"] / 1e3 / hbm,
           "gemm2_frac_of_%s_hbm" % src: b2 / us["moe_gemm2"] / 1e3 / hbm}
    native.assert_device_ok()
    print(json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in out.items()}))


if __name__ == "__main__":
    main()
