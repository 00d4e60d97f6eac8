"""Worker for the multi-rank tests (one process per rank, launched by torch.distributed.run).

cpu:  tiny model, gloo, TorchDistComm: rank logits must match the single-rank model.
cuda: flagship-shaped small model over the fused NVLink communicator, plus the collectives themselves against NCCL.
Writes 'OK' lines; any assertion failure exits non-zero.
"""
import argparse
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from helpers import MiniRunner  # noqa: E402
from minisgl.models import synth  # noqa: E402
from minisgl.models.config import ModelConfig  # noqa: E402
from minisgl.parallel.comm import TorchDistComm, init_distributed  # noqa: E402
from minisgl.parallel.info import DistributedInfo  # noqa: E402


def rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / b.float().cpu().norm()).item()


def main():
    """Runs the checks; a failing rank does not just exit: every rank first reaches the final barrier and tears its
    process group (and with it the symmetric / multicast mappings) down, then the failing one exits non-zero."""
    failure = None
    try:
        _checks()
    except BaseException as e:  # noqa: BLE001 - reported below, after the orderly teardown
        import traceback

        failure = e
        traceback.print_exc()
    try:
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception:  # pragma: no cover
        pass
    if failure is not None:
        sys.exit(1)


def _checks():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--moe-mode", default="ep")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    info = DistributedInfo(rank, world)
    g = torch.Generator().manual_seed(0)
    if args.device == "cpu":
        cfg = ModelConfig.tiny()
        dev = torch.device("cpu")
        _, comm = init_distributed(info, dev, vocab_size=cfg.vocab_size)
        assert isinstance(comm, TorchDistComm)
        toks = torch.randint(0, cfg.vocab_size, (90,), generator=g).tolist()
        tp = MiniRunner(cfg, "cpu", comm=comm, moe_mode=args.moe_mode, rank=rank, size=world, seed=1)
        l_tp = tp.step([(0, toks)])
        single = MiniRunner(cfg, "cpu", seed=1)
        l_1 = single.step([(0, toks)])
        assert rel(l_tp, l_1) < 0.08, rel(l_tp, l_1)  # bf16 partial sums + e4m3 rounding flips
        assert torch.equal(l_tp.argmax(-1), l_1.argmax(-1))
        print(f"OK cpu rank {rank} rel {rel(l_tp, l_1):.4f}", flush=True)
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        cfg = dataclasses.replace(ModelConfig.flash().with_layers(4), n_routed_experts=16, vocab_size=4096,
                                  n_hash_layers=1)
        _, comm = init_distributed(info, dev, vocab_size=cfg.vocab_size, max_rows=2048, hidden=cfg.hidden_size)
        from minisgl.ops import native, quant
        from minisgl.parallel.symm import SymmComm

        assert isinstance(comm, SymmComm), type(comm)
        assert comm.big, "the block-wise two-shot path failed its start-up check"
        assert comm.sp_min_rows > 0, "the row-sharded exchange failed its start-up check"
        if comm.has_multicast and os.environ.get("MINISGL_DISABLE_MULTIMEM", "0") != "1":
            assert comm.multimem, "the in-switch all-reduce failed its start-up check"
        print(f"rank {rank}: multicast {comm.has_multicast} multimem {comm.multimem} big {comm.big}", flush=True)
        # 1) stand-alone all-reduce vs NCCL, several sizes, repeated (epochs / parity buffers)
        # (2000 rows: more blocks than CTAs, i.e. several passes of the block-wise path)
        for rows in (1, 8, 128, 257, 1000, 2000):
            for it in range(3):
                x = (torch.randn(rows, 4096, device=dev, generator=None) * (rank + 1)).to(torch.bfloat16)
                ref = x.float().clone()
                dist.all_reduce(ref)
                out = comm.all_reduce(x)
                torch.cuda.synchronize()
                assert rel(out, ref) < 1e-2, (rows, it, rel(out, ref))
        # 1b) a rank that arrives half a second late (a host-side pause before its launch, as a GC pause or a slow
        # message would cause): the others wait inside their kernels, well within the limit, and the sums still agree
        for late in range(min(world, 2)):
            x = (torch.randn(128, 4096, device=dev) * (rank + 1)).to(torch.bfloat16)
            ref = x.float().clone()
            dist.all_reduce(ref)
            torch.cuda.synchronize()
            dist.barrier()
            if rank == late:
                import time

                time.sleep(0.5)
            out = comm.all_reduce(x)
            torch.cuda.synchronize()
            assert rel(out, ref) < 1e-2, ("late rank", late, rel(out, ref))
            assert native.read_status(clear=False)[0] == 0
        # 2) fused FP8 GEMM + all-reduce vs separate GEMM + NCCL
        from minisgl.ops import api as O

        for m in (1, 8, 128, 300, 1500):
            xx = torch.randn(m, 1024, device=dev).to(torch.bfloat16)
            ww = torch.randn(4096, 1024, device=dev) * 0.02
            wq, wsc = quant.fp8_weight_quant(ww)
            ws = quant.e8m0_decode(wsc)
            xq, sx = O.fp8_quant(xx)
            sep = O.gemm_fp8(xq, sx, wq, ws, out_dtype=torch.float32)
            dist.all_reduce(sep)
            fused = comm.gemm_fp8_allreduce(xq, sx, wq, ws)
            torch.cuda.synchronize()
            assert rel(fused, sep) < 1e-2, (m, rel(fused, sep))
        # every rank must hold bit-identical results
        chk = fused.float().sum().reshape(1).clone()
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert float(lo) == float(hi)
        # 2b) greedy sampling over vocabulary-parallel logits: per-shard argmax + in-kernel candidate exchange must
        # give the argmax of the gathered row on every rank, ties to the lowest token id
        vl = 4096 // world
        gen = torch.Generator().manual_seed(99)
        full = torch.randn(128, 4096, generator=gen)
        full[5, 100] = full[5, 4000] = 60.0
        shard = full[:, rank * vl:(rank + 1) * vl].contiguous().to(dev)
        from minisgl.models.deepseek_v4 import GreedyTail

        fbuf = torch.zeros(200, dtype=torch.int32, device=dev)
        sl = torch.arange(128, dtype=torch.int32, device=dev)
        for it in range(3):
            toks = comm.greedy_tokens(shard, sl, None, GreedyTail(fbuf))
            torch.cuda.synchronize()
            want = full.argmax(-1)
            want[5] = 100
            assert toks.cpu().tolist() == want.tolist(), (it, (toks.cpu() != want).nonzero().flatten()[:5])
            assert fbuf[:128].cpu().tolist() == want.tolist()
        # 2c) row-sharded exchange, kernel by kernel.  All-gather fused into a GEMM's loads: every rank writes only its
        # own rows of a common tensor into the gathered buffer, pushes them, and the gated GEMM over ALL rows must
        # equal the plain GEMM over the full tensor.  Reduce-scatter fused into a GEMM epilogue: against NCCL.
        from minisgl.ops.gemm import gemm_fp8_gated
        from minisgl.parallel.symm import SpPlan

        for trows in (600, 1500):
            plan = SpPlan(trows, rank, world)
            gen = torch.Generator().manual_seed(7 + trows)
            xf = torch.randn(trows, 4096, generator=gen).to(torch.bfloat16).to(dev)
            xq_full, sx_full = O.fp8_quant(xf)
            ag_y, ag_q, ag_s = comm.sp_buffers(plan, comm.CH_ATTN)
            ag_y.zero_(); ag_q.view(torch.uint8).zero_(); ag_s.zero_()
            r0, n = plan.row0, plan.n_own
            ag_y[r0:r0 + n] = xf[r0:r0 + n]
            ag_q[r0:r0 + n] = xq_full[r0:r0 + n]
            ag_s[r0:r0 + n] = sx_full[r0:r0 + n]
            torch.cuda.synchronize()
            dist.barrier()
            ww = torch.randn(2048, 4096, device=dev) * 0.02
            wq, wsc = quant.fp8_weight_quant(ww)
            ws = quant.e8m0_decode(wsc)
            gate = comm.sp_all_gather(plan, comm.CH_ATTN)
            got = gemm_fp8_gated(ag_q[:trows], ag_s[:trows], wq, ws, gate)
            want = O.gemm_fp8(xq_full, sx_full, wq, ws)
            torch.cuda.synchronize()
            assert torch.equal(got, want), ("gated gemm", trows, rel(got, want))
            assert torch.equal(ag_y[:trows], xf), "gathered bf16 rows differ"
            # reduce-scatter epilogue
            xr = (torch.randn(trows, 1024, device=dev) * (rank + 1)).to(torch.bfloat16)
            xq, sx = O.fp8_quant(xr)
            w2 = torch.randn(4096, 1024, device=dev) * 0.02
            w2q, w2c = quant.fp8_weight_quant(w2)
            w2s = quant.e8m0_decode(w2c)
            full = O.gemm_fp8(xq, sx, w2q, w2s, out_dtype=torch.float32)
            dist.all_reduce(full)
            for push in (False, True):          # in-switch form (where a multicast mapping exists) and peer-store form
                own = comm.sp_gemm_fp8_reduce_scatter(plan, comm.CH_ATTN, xq, sx, w2q, w2s, push=push)
                torch.cuda.synchronize()
                assert own.shape[0] == n
                if n:
                    assert rel(own, full[r0:r0 + n]) < 1e-2, ("reduce-scatter", push, trows,
                                                                rel(own, full[r0:r0 + n]))
            assert native.read_status(clear=False)[0] == 0
        # 3) whole model: tensor/expert parallel vs single rank
        # (600 prompt tokens: the prefill's collectives take the block-wise path, the decode steps the row-wise one)
        toks = torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist()
        kw = dict(page_size=256, num_pages=8, num_slots=2, max_len=1024)
        tp = MiniRunner(cfg, dev, comm=comm, moe_mode=args.moe_mode, rank=rank, size=world, seed=2, **kw)
        l_tp = tp.step([(0, toks)])
        for t in toks[:3]:
            l_tp = tp.step([(0, [t])])
        single = MiniRunner(cfg, dev, seed=2, **kw)
        l_1 = single.step([(0, toks)])
        for t in toks[:3]:
            l_1 = single.step([(0, [t])])
        torch.cuda.synchronize()
        native.assert_device_ok()
        assert rel(l_tp, l_1) < 0.2, rel(l_tp, l_1)  # e4m3 rounding and router top-k flips amplify over layers
        # 3b) the same prompt with the layer row-sharded during prefill (reduce-scatter / all-gather instead of the
        # all-reduces): same logits as the replicated run up to bf16 summation order
        assert comm.counters["sp_all_gather"] == 2, comm.counters      # only the kernel checks above used it so far
        comm.sp_min_rows = 256
        sp = MiniRunner(cfg, dev, comm=comm, moe_mode=args.moe_mode, rank=rank, size=world, seed=2, **kw)
        l_sp = sp.step([(0, toks)])
        for t in toks[:3]:
            l_sp = sp.step([(0, [t])])
        torch.cuda.synchronize()
        native.assert_device_ok()
        assert comm.counters["sp_all_gather"] == 2 + 2 * cfg.num_layers, comm.counters
        assert rel(l_sp, l_tp) < 0.2, ("row-sharded vs replicated", rel(l_sp, l_tp))   # same bound as sharded vs single
        assert rel(l_sp, l_1) < 0.2, rel(l_sp, l_1)
        # 3c) a prompt so short that the last rank owns no row at all (one 128-row block for the whole prompt)
        comm.sp_min_rows = 64
        short = toks[:100]
        s_sp = MiniRunner(cfg, dev, comm=comm, moe_mode=args.moe_mode, rank=rank, size=world, seed=2, **kw)
        l_short = s_sp.step([(0, short)])
        comm.sp_min_rows = 0
        s_tp = MiniRunner(cfg, dev, comm=comm, moe_mode=args.moe_mode, rank=rank, size=world, seed=2, **kw)
        l_short_tp = s_tp.step([(0, short)])
        torch.cuda.synchronize()
        native.assert_device_ok()
        assert rel(l_short, l_short_tp) < 0.2, ("short row-sharded prompt", rel(l_short, l_short_tp))
        comm.sp_min_rows = 1024
        print(f"OK cuda rank {rank} rel {rel(l_tp, l_1):.4f} counters {comm.counters}", flush=True)


if __name__ == "__main__":
    main()
