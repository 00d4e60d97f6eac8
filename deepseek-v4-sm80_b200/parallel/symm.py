"""Communicator whose collectives run *inside* this library's kernels over NVLink peer memory.

One symmetric allocation per rank (``torch.distributed._symmetric_memory``: CUDA VMM + handle exchange, every peer's
base pointer visible to every rank) holds flag words and double-buffered partial-result areas for three channels:

  channel 0  attention output projection: ``wo_b`` FP8 GEMM whose epilogue all-reduces (csrc/gemm_tcgen05.cu)
  channel 1  MoE combine: per-token route sum + shared expert, all-reduced in the same kernel (csrc/moe.cu)
  channel 2  generic stand-alone all-reduce (csrc/comm.cu)

The protocol (epochs, parity buffers, bounded waits) is documented in csrc/comm.cuh.  The logits all-gather, which
runs once per forward, stays on NCCL.  This replaces the reference's PyNCCL object
(python/minisgl/kernel/csrc/src/pynccl.cu:73-176: copy-in, ncclAllReduce on a registered window, copy-out).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..models.deepseek_v4 import Comm
from ..ops import native as nv
from ..ops.native import I
from .info import DistributedInfo

# Diagnosis only (MINISGL_SKIP_EXCHANGE=1): run the two fused call sites without their peer exchange, to read the
# cost of the collectives off a benchmark.  The results are then wrong (each rank keeps its partial sums).
import os as _os

_SKIP_EXCHANGE = _os.environ.get("MINISGL_SKIP_EXCHANGE", "0") == "1"
# MINISGL_BIG_ALLREDUCE=0 keeps large tensors (prefill) on the one-shot exchange; with it on, tensors of more than
# MINISGL_BIG_MIN_ROWS rows take the block-wise two-shot path (the one-shot form moves world-1 times the tensor out of
# every GPU, the two-shot form (world-1)/world of it, at the price of a second flag round trip).
_BIG = _os.environ.get("MINISGL_BIG_ALLREDUCE", "1") == "1"
_BIG_MIN_ROWS = max(int(_os.environ.get("MINISGL_BIG_MIN_ROWS", "128")), 1)

MAX_RANKS = 8


class CommCtx(ctypes.Structure):
    _fields_ = [("peer", ctypes.c_void_p * MAX_RANKS), ("rank", ctypes.c_int), ("world", ctypes.c_int),
                ("channel", ctypes.c_int), ("big", ctypes.c_int), ("data_bytes", ctypes.c_longlong),
                ("small_bytes", ctypes.c_longlong),
                ("epoch", ctypes.c_void_p), ("done", ctypes.c_void_p),
                ("mc", ctypes.c_void_p), ("mm", ctypes.c_int), ("pad_", ctypes.c_int)]


class SpCtx(ctypes.Structure):
    """Mirror of the native SpCtx (csrc/comm.cuh): one row-sharded exchange on one channel."""

    _fields_ = [("peer", ctypes.c_void_p * MAX_RANKS), ("mc", ctypes.c_void_p), ("rank", ctypes.c_int),
                ("world", ctypes.c_int), ("rows_per_rank", ctypes.c_int), ("hidden", ctypes.c_int),
                ("flags_off", ctypes.c_longlong), ("ag_off", ctypes.c_longlong), ("rs_off", ctypes.c_longlong),
                ("seq", ctypes.c_uint), ("use_mc", ctypes.c_int)]


class SpPlan:
    """Row ownership of one forward of ``t`` rows: rank r owns rows [r * rpr, (r + 1) * rpr) with rpr a multiple of
    128 (the GEMM row tile), ``tpad = world * rpr``; ``row0`` / ``n_own`` describe this rank's valid rows."""

    def __init__(self, t: int, rank: int, world: int):
        self.t = t
        self.rpr = -(-(-(-t // world)) // 128) * 128
        self.tpad = self.rpr * world
        self.row0 = min(rank * self.rpr, t)
        self.n_own = max(min(t - rank * self.rpr, self.rpr), 0)


class SymmComm(Comm):
    fused = True
    CH_ATTN, CH_MOE, CH_GENERIC = 0, 1, 2

    def __init__(self, info: DistributedInfo, device, vocab_size: Optional[int] = None, max_rows: int = 8192,
                 hidden: int = 4096, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        if info.size > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks are supported")
        self.rank, self.size, self.vocab_size = info.rank, info.size, vocab_size
        self.device = torch.device(device)
        self.group = group or dist.group.WORLD
        lib = nv.cuda_lib()
        fb, ch, sl, mr = ctypes.c_longlong(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        nv.check(lib.dsv4_comm_layout(ctypes.byref(fb), ctypes.byref(ch), ctypes.byref(sl), ctypes.byref(mr)),
                 "dsv4_comm_layout")
        assert mr.value == MAX_RANKS
        assert lib.dsv4_comm_ctx_size() == ctypes.sizeof(CommCtx), "CommCtx layout differs from the native library's"
        self.flags_bytes, self.channels, self.slots = fb.value, ch.value, sl.value
        # row-sharded exchange: rows are padded to world x (a multiple of 128)
        self.hidden = hidden
        self.sp_tpad_max = SpPlan(max_rows, 0, self.size).tpad
        assert lib.dsv4_sp_ctx_size() == ctypes.sizeof(SpCtx), "SpCtx layout differs from the native library's"
        self.sp_slots = lib.dsv4_sp_slots()
        self.data_bytes = (self.sp_tpad_max * hidden * 2 + 255) // 256 * 256
        # result buffers of the two-shot path (row counts of a decode batch): the owner of a row writes its sum here
        self.small_bytes = (min(max_rows, 256) * hidden * 2 + 255) // 256 * 256
        total = self.flags_bytes + self.channels * 2 * self.data_bytes + self.channels * 2 * self.small_bytes
        # appended for the row-sharded exchange: flag words, then one gathered buffer (bf16 rows | e4m3 rows | scales)
        # per layer block kind
        self.sp_flags_off = total
        total += (2 * MAX_RANKS * self.sp_slots * 4 + 255) // 256 * 256
        self.sp_ag_bytes = (self.sp_tpad_max * (3 * hidden + hidden // 128 * 4) + 255) // 256 * 256
        self.sp_ag_off = [total, total + self.sp_ag_bytes]
        total += 2 * self.sp_ag_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.buf.zero_()
        self.state = torch.zeros(2 * self.channels, dtype=torch.int32, device=self.device)  # epochs, done counters
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        off = int(getattr(self.handle, "offset", 0) or 0)     # of this tensor inside the rank's allocation block
        ptrs = [int(p) + off for p in self.handle.buffer_ptrs]
        if ptrs[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric-memory handle does not describe the buffer it was made for")
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.mc_ptr = mc + off if mc else 0
        self.has_multicast = bool(self.mc_ptr)
        self.ctx = []
        for c in range(self.channels):
            x = CommCtx()
            for r in range(self.size):
                x.peer[r] = ptrs[r]
            x.rank, x.world, x.channel, x.data_bytes = self.rank, self.size, c, self.data_bytes
            x.small_bytes = self.small_bytes
            x.epoch = self.state.data_ptr()
            x.done = self.state.data_ptr() + 4 * self.channels
            x.mc, x.mm = self.mc_ptr or None, 0
            self.ctx.append(x)
        self.counters = {"all_reduce": 0, "gemm_allreduce": 0, "moe_allreduce": 0, "all_gather": 0,
                         "sp_all_gather": 0, "sp_reduce_scatter": 0}
        self._ptrs = ptrs
        self.sp_seq = 0
        self.sp_counters = torch.zeros(2 * self.sp_slots, dtype=torch.int32, device=self.device)
        # rows at or above this count run the layer row-sharded (prefill); 0 switches it off
        self.sp_min_rows = int(_os.environ.get("MINISGL_SP_MIN_ROWS", "1024")) if self.size > 1 else 0
        if self.sp_tpad_max // 128 > self.sp_slots or hidden % 256:
            self.sp_min_rows = 0
        self.big = False
        self.multimem = False
        from ..env import ENV

        if self.has_multicast and self.size > 1 and not _SKIP_EXCHANGE and not ENV.DISABLE_MULTIMEM:
            self._enable_multimem(hidden, min(max_rows, 256))
        if _BIG and self.size > 1 and not _SKIP_EXCHANGE and max_rows >= 512:
            self._enable_big(hidden, max_rows)
        from ..utils.logger import init_logger

        if self.sp_min_rows > 0 and not _SKIP_EXCHANGE:
            self._check_sp(hidden, min(max_rows, 1024))
        init_logger(__name__).info_rank0(
            "NVLink communicator: %d ranks, multicast mapping %s, in-switch reductions %s, block-wise prefill path %s, "
            "row-sharded prefill %s", self.size, "yes" if self.has_multicast else "no",
            "on" if self.multimem else "off", "on" if self.big else "off",
            f"from {self.sp_min_rows} rows" if self.sp_min_rows > 0 else "off")

    @property
    def mode(self) -> str:
        return ("multimem" if self.multimem else "p2p") + ("+blockwise" if self.big else "")

    def _set_big(self, on: bool) -> None:
        self.big = on
        for x in self.ctx:
            x.big = _BIG_MIN_ROWS if on else 0

    def _check_sp(self, hidden: int, rows: int) -> None:
        """Start-up check of the row-sharded exchange on this machine and world size: an all-gather push followed by
        a gated GEMM must reproduce the plain GEMM over the full tensor bit for bit, and a reduce-scatter GEMM must
        agree with GEMM + NCCL.  A failure (or a wait that ran out) switches the row-sharded prefill off on all ranks
        together; prefill then keeps replicated activations and the all-reduce paths."""
        from ..ops import api as O
        from ..ops import quant
        from ..ops.gemm import gemm_fp8_gated
        from ..utils.logger import init_logger

        rows = rows - rows % 8 + 5            # ragged: the last row block is partial, the last rank may own less
        plan = SpPlan(rows, self.rank, self.size)
        good = plan.tpad <= self.sp_tpad_max
        status = [0]
        if good:
            g = torch.Generator(device="cpu").manual_seed(777)                 # the same tensor on every rank
            xf = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(self.device)
            w = (torch.randn(256, hidden, generator=g) * 0.02).to(self.device)
            wq, wc = quant.fp8_weight_quant(w)
            ws = quant.e8m0_decode(wc)
            xq, sx = O.fp8_quant(xf)
            ag_y, ag_q, ag_s = self.sp_buffers(plan, self.CH_ATTN)
            r0, n = plan.row0, plan.n_own
            ag_y[r0:r0 + n] = xf[r0:r0 + n]
            ag_q[r0:r0 + n] = xq[r0:r0 + n]
            ag_s[r0:r0 + n] = sx[r0:r0 + n]
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            gate = self.sp_all_gather(plan, self.CH_ATTN)
            got = gemm_fp8_gated(ag_q[:rows], ag_s[:rows], wq, ws, gate)
            want = O.gemm_fp8(xq, sx, wq, ws, splits=1)       # the gated GEMM does not split K: same summation order
            torch.cuda.synchronize(self.device)
            good = bool(torch.equal(got, want)) and bool(torch.equal(ag_y[:rows], xf))
            # reduce-scatter: every rank contributes a different K shard
            g2 = torch.Generator(device="cpu").manual_seed(900 + self.rank)
            xr = torch.randn(rows, 512, generator=g2).to(torch.bfloat16).to(self.device)
            w2 = (torch.randn(hidden, 512, generator=g2) * 0.02).to(self.device)
            w2q, w2c = quant.fp8_weight_quant(w2)
            w2s = quant.e8m0_decode(w2c)
            xq2, sx2 = O.fp8_quant(xr)
            full = O.gemm_fp8(xq2, sx2, w2q, w2s, out_dtype=torch.float32)
            dist.all_reduce(full, group=self.group)
            own = self.sp_gemm_fp8_reduce_scatter(plan, self.CH_ATTN, xq2, sx2, w2q, w2s)
            torch.cuda.synchronize(self.device)
            status = nv.read_status(clear=True)
            if n > 0:
                ref = full[r0:r0 + n]
                good = good and float((own.float() - ref).abs().max()) <= 0.02 * float(ref.abs().max()) + 1e-3
            good = good and status[0] == 0
        flag = torch.tensor([1 if good else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self.sp_min_rows = 0
            init_logger(__name__).warning("row-sharded exchange failed its start-up check (status %s); prefill keeps "
                                          "replicated activations", status[:4])
        self.counters["sp_all_gather"] = self.counters["sp_reduce_scatter"] = 0

    def _set_multimem(self, on: bool) -> None:
        self.multimem = on
        for x in self.ctx:
            x.mm = 1 if on else 0

    def _enable_multimem(self, hidden: int, rows: int) -> None:
        """Switch the in-switch (NVLS) reductions on and keep them only if, on a few random tensors, (a) the sums
        agree with NCCL, (b) no wait ran out and (c) every rank received exactly the same bits -- the one-shot form
        lets each rank ask the switch for the sum itself, and replicated activations must stay identical across
        ranks.  All ranks decide together."""
        from ..utils.logger import init_logger

        self._set_multimem(True)
        good = True
        status = [0]
        for it in range(3):
            g = torch.Generator(device="cpu").manual_seed(4321 + 17 * it + self.rank)
            x = (torch.randn(rows, hidden, generator=g) * (1 + it)).to(self.device, torch.bfloat16)
            want = x.float()
            dist.all_reduce(want, group=self.group)
            got = self.all_reduce(x)
            torch.cuda.synchronize(self.device)
            status = nv.read_status(clear=True)
            tol = 0.03 * self.size ** 0.5 * 4 * (1 + it)
            bits = got.view(torch.int16).to(torch.int64)
            h = torch.stack([bits.sum(), (bits * torch.arange(1, bits.numel() + 1, device=self.device).view_as(bits)
                                          % 1000003).sum()])
            lo, hi = h.clone(), h.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
            good = good and status[0] == 0 and bool(torch.isfinite(got).all()) and \
                float((got.float() - want).abs().max()) < tol and bool((lo == hi).all())
        flag = torch.tensor([1 if good else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self._set_multimem(False)
            init_logger(__name__).warning("in-switch (multimem) all-reduce failed its start-up check "
                                          f"(status {status[:4]}); using the peer-to-peer exchange")
        self.counters["all_reduce"] = 0

    def _enable_big(self, hidden: int, max_rows: int) -> None:
        """Switch the block-wise two-shot path on, reduce tensors with it and with NCCL, and keep it only if every
        rank saw the same sums and no wait ran out (otherwise all ranks fall back to the one-shot exchange together).
        Checked sizes: ``max_rows`` rows -- the largest prefill forward, with more 8-row blocks than CTAs, so
        that every CTA runs several passes and the owner of its blocks rotates through all ranks --, a ragged
        row count that ends in a partial block, and the smallest tensor that takes this path."""
        from ..utils.logger import init_logger

        good, status = True, [0]
        self._set_big(True)
        for rows in (max_rows, max(max_rows // 2 - 3, 257), _BIG_MIN_ROWS + 1):
            g = torch.Generator(device="cpu").manual_seed(1234 + self.rank)
            x = torch.randn(rows, hidden, generator=g).to(self.device, torch.bfloat16)
            want = x.float()
            dist.all_reduce(want, group=self.group)
            got = self.all_reduce(x)
            torch.cuda.synchronize(self.device)
            status = nv.read_status(clear=True)
            tol = 0.03 * self.size ** 0.5 * 4      # bf16 rounding of sums of `size` unit normals
            good = good and status[0] == 0 and bool(torch.isfinite(got).all()) and \
                float((got.float() - want).abs().max()) < tol
            del x, want, got
        flag = torch.tensor([1 if good else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self._set_big(False)
            init_logger(__name__).warning("block-wise two-shot all-reduce failed its start-up check "
                                          f"(status {status[:4]}); prefill uses the one-shot exchange")
        self.counters["all_reduce"] = 0

    # ------------------------------------------------------------------ row-sharded (sequence-parallel) exchange
    def sp_plan(self, t: int) -> Optional[SpPlan]:
        """Ownership plan if a forward of t rows should run row-sharded, else None."""
        if self.sp_min_rows <= 0 or t < self.sp_min_rows or _SKIP_EXCHANGE:
            return None
        p = SpPlan(t, self.rank, self.size)
        return p if p.tpad <= self.sp_tpad_max else None

    def _sp_ctx(self, plan: SpPlan, channel: int, seq: int) -> SpCtx:
        c = SpCtx()
        for r in range(self.size):
            c.peer[r] = self._ptrs[r]
        c.mc = self.mc_ptr or None
        c.rank, c.world, c.rows_per_rank, c.hidden = self.rank, self.size, plan.rpr, self.hidden
        c.flags_off, c.ag_off = self.sp_flags_off, self.sp_ag_off[channel]
        c.rs_off = self.flags_bytes + (channel * 2) * self.data_bytes       # parity-0 area of the channel
        c.seq, c.use_mc = seq, 1 if (self.multimem and self.mc_ptr) else 0
        return c

    def sp_buffers(self, plan: SpPlan, channel: int):
        """This rank's copy of the channel's gathered buffer: (y bf16 [tpad, h], q e4m3 [tpad, h], s fp32 [tpad, h/128])."""
        h, tp = self.hidden, plan.tpad
        o = self.sp_ag_off[channel]
        y = self.buf[o:o + tp * h * 2].view(torch.bfloat16).view(tp, h)
        o += tp * h * 2
        q = self.buf[o:o + tp * h].view(torch.float8_e4m3fn).view(tp, h)
        o += tp * h
        s = self.buf[o:o + tp * (h // 128) * 4].view(torch.float32).view(tp, h // 128)
        return y, q, s

    def sp_all_gather(self, plan: SpPlan, channel: int) -> SpCtx:
        """Pushes this rank's rows of the gathered buffer (written by the kernels before this call) to all peers and
        returns the context with which the consuming GEMMs gate their loads."""
        self.sp_seq += 1
        self.counters["sp_all_gather"] += 1
        ctx = self._sp_ctx(plan, channel, self.sp_seq)
        nv.call("sp_ag_push", ctypes.byref(ctx), I(plan.tpad), nv.ptr(self.sp_counters))
        return ctx

    def sp_gemm_fp8_reduce_scatter(self, plan: SpPlan, channel: int, xq, sx, w, ws, hc=None,
                                   push: bool = False) -> torch.Tensor:
        """Projection of all rows by this rank's K shard, reduce-scattered: the GEMM epilogue stores every partial row
        into its owner's buffer over NVLink, the owner adds the ranks' partials.  Returns this rank's rows
        [n_own, n], or with hc = (residual, post, comb) of the own rows the new residual streams [n_own, 4, n].
        Two forms: with a multicast mapping the epilogue leaves the partial tile in the rank's own buffer and the
        owner's reduction is a ``multimem.ld_reduce`` (the switch adds the ranks' copies); ``push=True`` or no multicast:
        the epilogue stores every partial row straight into its owner's buffer and the owner adds them."""
        m, k = xq.shape
        n = w.shape[0]
        self.sp_seq += 1
        self.counters["sp_reduce_scatter"] += 1
        ctx = self._sp_ctx(plan, channel, self.sp_seq)
        if push:
            ctx.use_mc = 0      # the epilogue stores the partial rows into the owners' buffers (no multicast needed)
        cnt = self.sp_counters[self.sp_slots:]
        nv.call("gemm_fp8_rs", nv.ptr(xq), nv.ptr(w), nv.ptr(sx), nv.ptr(ws), I(m), I(n), I(k), I(xq.stride(0)),
                I(w.stride(0)), I(0), ctypes.byref(ctx), nv.ptr(cnt))
        # with a multicast mapping the GEMM leaves its partial in its own buffer and the owner's reduction asks the
        # switch for the sum; otherwise the epilogue stored the partial rows into the owners' buffers
        return self._sp_reduce(ctx, plan, n, hc, mc_mode=1 if ctx.use_mc else 0)

    def sp_moe_finalize_reduce_scatter(self, plan: SpPlan, rows, moe_plan, max_tiles, shared, t, topk, h, hc=None):
        """Expert combine of all rows on this rank's experts (+ shared expert shard), reduce-scattered like above."""
        self.sp_seq += 1
        self.counters["sp_reduce_scatter"] += 1
        ctx = self._sp_ctx(plan, self.CH_MOE, self.sp_seq)
        cnt = self.sp_counters[self.sp_slots:]
        nv.call("moe_finalize_rs", nv.ptr(rows), nv.ptr(moe_plan), I(t * topk), I(max_tiles), nv.ptr(shared), I(t),
                I(topk), I(h), ctypes.byref(ctx), nv.ptr(cnt))
        return self._sp_reduce(ctx, plan, h, hc)

    def _sp_reduce(self, ctx: SpCtx, plan: SpPlan, n: int, hc, mc_mode: int = 0):
        if hc is not None:
            res, post, comb = hc
            xout = torch.empty_like(res)
            nv.call("sp_rs_reduce", ctypes.byref(ctx), I(plan.n_own), I(n), nv.ptr(None), nv.ptr(res), nv.ptr(post),
                    nv.ptr(comb), nv.ptr(xout), I(mc_mode))
            return xout
        out = torch.empty(plan.n_own, n, dtype=torch.bfloat16, device=self.device)
        nv.call("sp_rs_reduce", ctypes.byref(ctx), I(plan.n_own), I(n), nv.ptr(out), nv.ptr(None), nv.ptr(None),
                nv.ptr(None), nv.ptr(None), I(mc_mode))
        return out

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor, tag: str = "") -> torch.Tensor:
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 2
        self.counters["all_reduce"] += 1
        out = torch.empty_like(x)
        nv.call("allreduce", nv.ptr(x), nv.ptr(out), I(x.shape[0]), I(x.shape[1]), nv.ptr(None), nv.ptr(None),
                nv.ptr(None), nv.ptr(None), ctypes.byref(self.ctx[self.CH_GENERIC]))
        return out

    def gemm_fp8_allreduce(self, xq, sx, w, ws, bn: int = 0, hc=None) -> torch.Tensor:
        """out = all_reduce(xq @ w^T).  The GEMM deposits its partial product in the channel's symmetric buffer and the
        all-reduce kernel follows as its programmatic dependent: row-wise for small tensors (decode; its peer reads are
        whole rows, the GEMM epilogue's would be 64-byte pieces of 128 x 32 tiles), block-wise two-shot above
        (prefill; 2 * (world-1)/world of the tensor crosses NVLink per rank instead of world-1 times the tensor).
        With the block-wise path off, large tensors are reduced in the GEMM's epilogue.
        hc = (residual, post, comb): the hyper-connection post mix is applied to the reduced rows by the same kernel
        and the new residual streams [m, 4, n] are returned."""
        m, k = xq.shape
        n = w.shape[0]
        self.counters["gemm_allreduce"] += 1
        if _SKIP_EXCHANGE:
            from ..ops import api as O

            y = O.gemm_fp8(xq, sx, w, ws)
            return O.hc_post(y, *hc) if hc is not None else y
        ctx = ctypes.byref(self.ctx[self.CH_ATTN])
        if m <= 256 or self.big:
            nv.call("gemm_fp8_allreduce", nv.ptr(xq), nv.ptr(w), nv.ptr(None), nv.ptr(sx), nv.ptr(ws), I(m), I(n), I(k),
                    I(xq.stride(0)), I(w.stride(0)), ctx, I(bn), I(1))
            if hc is not None:
                res, post, comb = hc
                xout = torch.empty_like(res)
                nv.call("allreduce", nv.ptr(None), nv.ptr(None), I(m), I(n), nv.ptr(res), nv.ptr(post), nv.ptr(comb),
                        nv.ptr(xout), ctx)
                return xout
            out = torch.empty(m, n, dtype=torch.bfloat16, device=xq.device)
            nv.call("allreduce", nv.ptr(None), nv.ptr(out), I(m), I(n), nv.ptr(None), nv.ptr(None), nv.ptr(None),
                    nv.ptr(None), ctx)
            return out
        out = torch.empty(m, n, dtype=torch.bfloat16, device=xq.device)
        nv.call("gemm_fp8_allreduce", nv.ptr(xq), nv.ptr(w), nv.ptr(out), nv.ptr(sx), nv.ptr(ws), I(m), I(n), I(k),
                I(xq.stride(0)), I(w.stride(0)), ctx, I(bn), I(0))
        if hc is not None:
            from ..ops import api as O

            return O.hc_post(out, *hc)
        return out

    def gemm_bf16_allreduce(self, x, w, bn: int = 0, channel: Optional[int] = None) -> torch.Tensor:
        m, k = x.shape
        n = w.shape[0]
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
        nv.call("gemm_bf16_allreduce", nv.ptr(x), nv.ptr(w), nv.ptr(out), I(m), I(n), I(k), I(x.stride(0)),
                I(w.stride(0)), ctypes.byref(self.ctx[self.CH_ATTN if channel is None else channel]), I(bn))
        return out

    def moe_finalize_allreduce(self, rows, plan, max_tiles, shared, num_valid, t, topk, h, hc=None) -> torch.Tensor:
        """hc = (residual, post, comb): the hyper-connection post mix is applied to the reduced rows in the same
        kernel and the new residual streams [t, 4, h] are returned."""
        self.counters["moe_allreduce"] += 1
        if _SKIP_EXCHANGE:
            from ..ops import cuda as C

            return C.moe_finalize(rows, plan, max_tiles, shared, num_valid, t, topk, h, hc)
        if hc is not None:
            res, post, comb = hc
            xout = torch.empty_like(res)
            nv.call("moe_finalize_allreduce", nv.ptr(rows), nv.ptr(plan), I(t * topk), I(max_tiles), nv.ptr(shared),
                    nv.ptr(None), nv.ptr(num_valid), I(t), I(topk), I(h), nv.ptr(res), nv.ptr(post), nv.ptr(comb),
                    nv.ptr(xout), ctypes.byref(self.ctx[self.CH_MOE]))
            return xout
        out = torch.empty(t, h, dtype=rows.dtype, device=rows.device)
        nv.call("moe_finalize_allreduce", nv.ptr(rows), nv.ptr(plan), I(t * topk), I(max_tiles), nv.ptr(shared),
                nv.ptr(out), nv.ptr(num_valid), I(t), I(topk), I(h), nv.ptr(None), nv.ptr(None), nv.ptr(None),
                nv.ptr(None), ctypes.byref(self.ctx[self.CH_MOE]))
        return out

    def greedy_tokens(self, logits_local, slots, num_valid, tail) -> torch.Tensor:
        """Per-shard argmax + candidate exchange + pick, in one kernel (csrc/comm.cu: greedy_tokens_kernel); no
        logits all-gather."""
        from ..ops import api as O

        self.counters["greedy_exchange"] = self.counters.get("greedy_exchange", 0) + 1
        per = -(-self.vocab_size // self.size) if self.vocab_size else logits_local.shape[1]
        return O.greedy_tokens(logits_local, self.rank * per, slots, num_valid, tail.token_feedback, tail.out,
                               comm_ctx=self.ctx[self.CH_GENERIC])

    def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
        self.counters["all_gather"] += 1
        b, vl = x.shape
        out = torch.empty(self.size * b, vl, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        full = out.view(self.size, b, vl).permute(1, 0, 2).reshape(b, self.size * vl)
        return full[:, : self.vocab_size] if self.vocab_size else full

    def barrier(self) -> None:
        dist.barrier(group=self.group)
