"""Microbenchmark of the fused compute+collective kernels against "NCCL all-reduce + separate kernel".

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m minisgl.benchmark.collectives

For M in {1, 8, 32, 128, 256, 8192} rows of hidden size 4096 (bf16 activations, N(0,1) inputs), per-rank shards of the
full model's shapes:
  * all_reduce        : the stand-alone in-kernel all-reduce vs ``dist.all_reduce`` (NCCL)
  * wo_b              : FP8 output projection [M, 8192/N] x [4096, 8192/N]^T with the all-reduce fused into the GEMM
                        epilogue vs the same GEMM followed by NCCL
  * moe_combine       : expert-parallel routed experts (256/N experts per rank, uniform-random top-6 routing), with the
                        per-token route sum + shared expert + all-reduce in one kernel vs unfused finalize + NCCL
  * wo_b_rs           : the same projection with the reduce-scatter fused into the GEMM epilogue (partial rows stored
                        straight into their owner's buffer, owner adds them) vs GEMM + ``dist.reduce_scatter_tensor``
  * ag_wqkv_a         : all-gather fused into the first projection [M, 4096] x [2048, 4096]^T (owners push their rows,
                        the GEMM's loads wait per 128-row block) vs ``dist.all_gather_into_tensor`` + GEMM
  * moe_rs            : the expert combine with the reduce-scatter form
Times of the first three are per call inside a CUDA graph of `--iters` calls (no host launch gaps), with an L2 flush
before every call whose own cost is subtracted, reduced with MAX over ranks.  The row-sharded forms (``*_rs``,
``ag_*``) number their exchanges on the host, so they and their NCCL baselines are timed eagerly, back to back on
one stream (marked ``eager`` in the output; below a few hundred rows such a number is bound by the host's launch
rate).  The roofline of a fused call is the slower of FLOPs / measured GEMM peak (twice the measured bf16 figure for
the e4m3 GEMMs) and the NVLink bytes per direction and GPU / 770 GB/s: all-reduce and reduce-scatter
(N-1)/N * M * 4096 * 2 (what the in-switch forms move; the one-shot peer-to-peer form moves N-1 times the tensor),
all-gather (N-1)/N * M * (4096 * 3 + 128) (bf16 rows, e4m3 rows and scales).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        j = json.load(open(path))
        return j["bf16_tflops"], j["hbm_gbs"], "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def _time(fn, iters, flush):
    """Microseconds per call, max over ranks.  `iters` calls are captured in one CUDA graph (as the engine runs
    them: no host launch gaps) together with an L2 flush before each when `flush` is set; the flush-only graph is
    timed too and subtracted."""
    from minisgl.benchmark.perf import flush_l2

    def graph_ms(body):
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            for _ in range(2):
                body()
        st.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(iters):
                body()
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 3

    if flush:
        def body():
            flush_l2()
            fn()
        ms = graph_ms(body) - graph_ms(flush_l2)
    else:
        ms = graph_ms(fn)
    t = torch.tensor([ms * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _time_eager(fn, iters):
    """Microseconds per call, max over ranks: `iters` calls issued back to back on the current stream."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[1, 8, 32, 128, 256, 8192])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--allreduce-only", action="store_true",
                    help="time the all-reduce forms only (plain, behind wo_b, behind the MoE combine)")
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    from minisgl.ops import api as O
    from minisgl.ops import cuda as C
    from minisgl.ops import native, quant
    from minisgl.parallel.comm import init_distributed
    from minisgl.parallel.info import DistributedInfo

    _, comm = init_distributed(DistributedInfo(rank, world), dev, max_rows=max(max(a.rows), 512), hidden=4096)
    tflops, hbm, src = _peaks()
    H, KO = 4096, 8192 // world
    e_local, inter, topk = 256 // world, 2048, 6
    g = torch.Generator(device=dev).manual_seed(rank)
    w = torch.randn(H, KO, device=dev, generator=g) * 0.02
    wq, wsc = quant.fp8_weight_quant(w)
    ws = quant.e8m0_decode(wsc)
    w13 = torch.randint(0, 256, (e_local, 2 * inter, H // 2), device=dev, dtype=torch.uint8).view(torch.int8)
    s13 = torch.randint(119, 122, (e_local, 2 * inter, H // 32), device=dev, dtype=torch.uint8)
    w2 = torch.randint(0, 256, (e_local, H, inter // 2), device=dev, dtype=torch.uint8).view(torch.int8)
    s2 = torch.randint(119, 122, (e_local, H, inter // 32), device=dev, dtype=torch.uint8)
    rows_out = []
    for m in a.rows:
        x = torch.randn(m, H, device=dev, generator=g).to(torch.bfloat16)
        xo = torch.randn(m, KO, device=dev, generator=g).to(torch.bfloat16)
        xq, sx = O.fp8_quant(xo)
        gi = torch.Generator(device=dev).manual_seed(1234)  # identical routing on every rank
        idx = torch.stack([torch.randperm(256, device=dev, generator=gi)[:topk] for _ in range(min(m, 512))])
        idx = idx.repeat((m + idx.shape[0] - 1) // idx.shape[0], 1)[:m].to(torch.int32).contiguous()
        wt = torch.rand(m, topk, device=dev, generator=gi)
        shared = torch.randn(m, H, device=dev, generator=g).to(torch.bfloat16)
        nccl_buf = x.clone()
        # bytes that must cross NVLink per direction and GPU for an all-reduce: every rank's partial leaves once except
        # for the part the rank reduces itself, and the reduced rows of the other ranks come back
        link_bytes = (world - 1) / world * m * H * 2
        t_link = link_bytes / (NVLINK_GBS * 1e3)  # us
        big_min = int(comm.ctx[0].big) if getattr(comm, "ctx", None) else 0
        res = {"rows": m, "world": world, "block_two_shot": bool(big_min and m > big_min)}
        res["allreduce_nccl_us"] = _time(lambda: dist.all_reduce(nccl_buf), a.iters, True)
        res["allreduce_ours_us"] = _time(lambda: comm.all_reduce(x), a.iters, True)

        def unfused_wo_b():
            y = O.gemm_fp8(xq, sx, wq, ws)
            dist.all_reduce(y)

        res["wo_b_gemm_plus_nccl_us"] = _time(unfused_wo_b, a.iters, True)
        res["wo_b_fused_us"] = _time(lambda: comm.gemm_fp8_allreduce(xq, sx, wq, ws), a.iters, True)
        flops = 2.0 * m * H * KO
        # e4m3 operands: the tensor pipe's nominal FP8 rate is twice its bf16 rate, so the compute floor is taken at
        # twice the measured bf16 GEMM throughput
        fp8_tflops = 2.0 * tflops
        res["wo_b_roofline_us"] = max(flops / (fp8_tflops * 1e6), t_link)
        res["wo_b_roofline_frac"] = res["wo_b_roofline_us"] / res["wo_b_fused_us"]
        base = rank * e_local

        def moe(fused):
            rows, plan, mt = C.moe_routed(x, idx, wt, w13, s13, w2, s2, 7.0, base, 256)
            if fused:
                return comm.moe_finalize_allreduce(rows, plan, mt, shared, None, m, topk, H)
            y = C.moe_finalize(rows, plan, mt, shared, None, m, topk, H)
            dist.all_reduce(y)
            return y

        res["moe_unfused_us"] = _time(lambda: moe(False), max(a.iters // 2, 3), True)
        res["moe_fused_us"] = _time(lambda: moe(True), max(a.iters // 2, 3), True)
        routes_local = m * topk / world
        moe_flops = routes_local * (2.0 * H * 2 * inter + 2.0 * inter * H)
        touched = e_local * (1 - (1 - 1 / 256) ** (m * topk)) if m * topk < 4096 else e_local
        moe_bytes = touched * (3 * inter * H // 2 + 3 * inter * H // 32)
        res["moe_roofline_us"] = max(moe_flops / (tflops * 1e6), moe_bytes / (hbm * 1e3), t_link)
        res["moe_roofline_frac"] = res["moe_roofline_us"] / res["moe_fused_us"]
        res["collectives"] = getattr(comm, "mode", "none")
        # ---- row-sharded forms (eager timing, see the module docstring)
        from minisgl.ops.gemm import gemm_fp8_gated
        from minisgl.parallel.symm import SpPlan

        plan = SpPlan(m, rank, world)
        if plan.tpad <= comm.sp_tpad_max and not a.allreduce_only:
            it = a.iters
            mp = plan.tpad
            pad_x = torch.zeros(mp, KO, device=dev, dtype=torch.bfloat16)
            pad_x[:m] = xo
            pq, ps_ = O.fp8_quant(pad_x)
            rs_out = torch.empty(plan.rpr, H, device=dev, dtype=torch.bfloat16)

            def rs_nccl():
                y = O.gemm_fp8(pq, ps_, wq, ws)
                dist.reduce_scatter_tensor(rs_out, y)

            res["wo_b_rs_gemm_plus_nccl_us"] = _time_eager(rs_nccl, it)
            res["wo_b_rs_fused_us"] = _time_eager(
                lambda: comm.sp_gemm_fp8_reduce_scatter(plan, comm.CH_ATTN, xq, sx, wq, ws), it)
            res["wo_b_rs_push_us"] = _time_eager(
                lambda: comm.sp_gemm_fp8_reduce_scatter(plan, comm.CH_ATTN, xq, sx, wq, ws, push=True), it)
            rs_link = (world - 1) / world * m * H * 2 / (NVLINK_GBS * 1e3)
            res["wo_b_rs_roofline_us"] = max(flops / (fp8_tflops * 1e6), rs_link)
            res["wo_b_rs_roofline_frac"] = res["wo_b_rs_roofline_us"] / res["wo_b_rs_fused_us"]
            # all-gather -> first projection (2048 output columns of the full model's wqkv_a)
            wa = torch.randn(2048, H, device=dev, generator=g) * 0.02
            waq, wac = quant.fp8_weight_quant(wa)
            was = quant.e8m0_decode(wac)
            ag_y, ag_q, ag_s = comm.sp_buffers(plan, comm.CH_ATTN)
            yq_own, ys_own = O.fp8_quant(torch.randn(plan.rpr, H, device=dev, generator=g).to(torch.bfloat16))
            ag_q[rank * plan.rpr:(rank + 1) * plan.rpr] = yq_own
            ag_s[rank * plan.rpr:(rank + 1) * plan.rpr] = ys_own
            full_q = torch.empty(mp, H, device=dev, dtype=torch.uint8)
            full_s = torch.empty(mp, H // 128, device=dev, dtype=torch.float32)
            full_y = torch.empty(mp, H, device=dev, dtype=torch.bfloat16)
            y_own = torch.randn(plan.rpr, H, device=dev, generator=g).to(torch.bfloat16)

            def ag_nccl():
                # the same three tensors the fused form delivers: the block's other consumers read the bf16 rows
                dist.all_gather_into_tensor(full_y, y_own)
                dist.all_gather_into_tensor(full_q, yq_own.view(torch.uint8))
                dist.all_gather_into_tensor(full_s, ys_own)
                O.gemm_fp8(full_q.view(torch.float8_e4m3fn)[:m], full_s[:m], waq, was)

            def ag_fused():
                gate = comm.sp_all_gather(plan, comm.CH_ATTN)
                gemm_fp8_gated(ag_q[:m], ag_s[:m], waq, was, gate)

            res["ag_wqkv_a_nccl_plus_gemm_us"] = _time_eager(ag_nccl, it)
            res["ag_wqkv_a_fused_us"] = _time_eager(ag_fused, it)
            ag_link = (world - 1) / world * m * (3 * H + H // 128 * 4) / (NVLINK_GBS * 1e3)
            res["ag_wqkv_a_roofline_us"] = max(2.0 * m * H * 2048 / (fp8_tflops * 1e6), ag_link)
            res["ag_wqkv_a_roofline_frac"] = res["ag_wqkv_a_roofline_us"] / res["ag_wqkv_a_fused_us"]

            def moe_rs():
                rows, mplan, mt = C.moe_routed(x, idx, wt, w13, s13, w2, s2, 7.0, base, 256)
                return comm.sp_moe_finalize_reduce_scatter(plan, rows, mplan, mt, shared, m, topk, H)

            res["moe_rs_fused_us"] = _time_eager(moe_rs, max(it // 2, 3))
            res["eager"] = ["wo_b_rs_*", "ag_wqkv_a_*", "moe_rs_*"]
        rows_out.append(res)
        if rank == 0:
            print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in res.items()}), flush=True)
    native.assert_device_ok()
    if rank == 0 and a.out:
        json.dump({"peaks": {"bf16_tflops": tflops, "hbm_gbs": hbm, "source": src, "nvlink_gbs": NVLINK_GBS},
                   "results": rows_out}, open(a.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
