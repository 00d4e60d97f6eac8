"""DeepSeek-V4 decoder: hyper-connected residual streams, MQA latent attention with a sliding window plus
C4 (indexer-selected) / C128 compressed history, and a routed + shared MoE.

The dataflow per layer follows the reference model (python/minisgl/models/deepseek_v4.py:753-922 for
attention, :1493-1523 for the MoE, :1614-1628 for the hyper-connection wrapper) but is written against the
operator facade :mod:`minisgl.ops.api`: on CUDA every call is a hand-written sm_100a kernel, on CPU the
fp32 PyTorch oracle.  Differences by design:

* dense FP8 weights are multiplied as FP8 on the tensor cores (activations quantised to e4m3 with the same
  power-of-two block scales the reference uses for its fake-quant), so no BF16 weight copies exist except
  ``wo_a``, whose input the model does not quantise;
* attention index surfaces are not materialised: kernels walk the request's page-table row;
* the embedding is replicated, so a forward has two reductions per layer and one all-gather at the head.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from ..ops import api as O
from ..ops.ref import RopeSpec
from .config import ModelConfig


@dataclass
class ForwardBatch:
    """Device-side description of one forward: T token rows belonging to B requests."""

    input_ids: torch.Tensor      # [T] int32
    positions: torch.Tensor      # [T] int32
    slots: torch.Tensor          # [T] int32 request table slot per row
    out_loc: torch.Tensor        # [T] int32 token location (page*page_size+offset); -1 = do not store
    last_idx: torch.Tensor       # [B] int64 rows whose logits are wanted
    page_table: torch.Tensor     # [slots+1, max_len] int32 token locations
    is_prefill: bool
    max_context: int             # max position + 1 over the batch (host value; bounds workspace widths)
    num_valid: Optional[torch.Tensor] = None  # [1] int32: rows >= num_valid are padding (graph replay)
    # [slots+1] int32 (decode only): the token of row t is token_feedback[slots[t]], the previous step's sample that
    # never left the device; the embedding kernel gathers it and fills input_ids
    token_feedback: Optional[torch.Tensor] = None


@dataclass
class GreedyTail:
    """Asks ``forward`` to finish with greedy sampling on the device: the argmax over the (vocabulary-parallel) logits
    is taken inside one kernel that also exchanges the shards' candidates between ranks, and the token goes to
    ``out[row]`` and to ``token_feedback[slot of the row]``.  The reference captures its greedy argmax in the decode
    graph for the same reason (python/minisgl/engine/graph.py:419-421)."""

    token_feedback: torch.Tensor   # [slots+1] int32
    out: Optional[torch.Tensor] = None  # [rows] int32 (allocated when None)
    logits_out: Optional[torch.Tensor] = None  # [rows, vocab / tp] fp32: where the head GEMM writes (else allocated)


class Comm:
    """Collectives the model needs; the single-rank default does nothing."""

    rank, size = 0, 1

    def all_reduce(self, x: torch.Tensor, tag: str = "") -> torch.Tensor:
        return x

    def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def greedy_tokens(self, logits_local, slots, num_valid, tail: "GreedyTail") -> torch.Tensor:
        """Greedy tokens of rows whose logits are sharded over the vocabulary; the default gathers, then picks."""
        return O.greedy_tokens(self.all_gather_last(logits_local), 0, slots, num_valid, tail.token_feedback, tail.out)


class DSV4Model:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], pool, comm: Optional[Comm] = None,
                 moe_mode: str = "tp"):
        self.cfg, self.w, self.pool = cfg, weights, pool
        self.comm = comm or Comm()
        self.moe_mode = moe_mode
        tp = self.comm.size
        assert cfg.num_heads % tp == 0 and cfg.o_groups % tp == 0, "tp must divide heads and o_groups"
        self.h_local = cfg.num_heads // tp
        self.g_local = cfg.o_groups // tp
        self.ropes = []
        for l in range(cfg.num_layers):
            r = cfg.ratio(l)
            base = cfg.compress_rope_theta if (r and cfg.compress_rope_theta is not None) else cfg.rope_theta
            self.ropes.append(RopeSpec.make(cfg.rope_head_dim, base, cfg.original_seq_len if r else 0,
                                            cfg.rope_factor, cfg.beta_fast, cfg.beta_slow))
        e_local = weights["L0.moe.w13"].shape[0]
        self.expert_base = self.comm.rank * e_local if (moe_mode == "ep" and tp > 1) else 0
        self.qat = cfg.nope_head_dim % 64 == 0
        if any(t.is_cuda for t in (weights["embed.weight"],)):
            from ..ops import native

            # the weights of this model are never written after loading: let the GEMMs fetch them ahead of the
            # dependent-launch wait
            native.check(native.cuda_lib().dsv4_gemm_set_weight_prefetch(1), "dsv4_gemm_set_weight_prefetch")
            from ..ops import cuda as C

            if C.MOE_KERNEL == "mx":
                # one-time re-tiling of the expert weights and scales for the block-scaled grouped GEMM (same bytes,
                # stage-contiguous order); the reference repacks its experts for Marlin at the same point
                # (python/minisgl/models/deepseek_v4.py:1718-1787)
                for l in range(cfg.num_layers):
                    C.prepare_experts(weights, f"L{l}.moe.")
        from ..env import ENV

        self._debug_bounds = bool(ENV.DEBUG_BOUNDS)  # audit every gathered index tensor before use
        self._side = None  # second CUDA stream for branches that do not depend on each other (created on first use)

    # ------------------------------------------------------------------ independent branches on a second stream
    def _fork(self, ref: torch.Tensor):
        """Context in which kernels go to the side stream, ordered after everything issued so far on the current
        stream.  The compressor / indexer-cache branch of attention and the shared expert do not depend on the main
        chain, and each of their kernels fills only part of the GPU, so they run beside it (also inside a captured
        CUDA graph, where the fork and the join become graph edges).  On CPU it is a no-op."""
        import contextlib

        if not ref.is_cuda or os.environ.get("MINISGL_SINGLE_STREAM", "0") == "1":
            return contextlib.nullcontext()
        if self._side is None:
            self._side = torch.cuda.Stream(device=ref.device)
        self._side.wait_stream(torch.cuda.current_stream(ref.device))
        return torch.cuda.stream(self._side)

    def _join(self, ref: torch.Tensor) -> None:
        if ref.is_cuda and self._side is not None and os.environ.get("MINISGL_SINGLE_STREAM", "0") != "1":
            torch.cuda.current_stream(ref.device).wait_stream(self._side)

    # ------------------------------------------------------------------ blocks
    def _fp8_linear(self, x, name: str, xq=None):
        if xq is None:
            xq = O.fp8_quant(x)
        return O.gemm_fp8(xq[0], xq[1], self.w[name + ".weight"], self.w[name + ".scale"])

    def attention(self, l: int, y: torch.Tensor, fb: ForwardBatch, yq=None, hc=None, sp=None) -> torch.Tensor:
        """hc = (residual, post, comb): when the communicator can fuse the hyper-connection post mix behind its
        reduction, the new residual streams are returned instead of the block output (flagged by ``self._mixed``).
        sp = (plan, gate): row-sharded layer.  y / yq are this rank's gathered buffer, whose rows arrive from their
        owners while the first projection runs (its loads wait per row block, ``gate``); the output projection is
        reduce-scattered and hc holds the own rows only."""
        cfg, w, p = self.cfg, self.w, f"L{l}.attn."
        t = y.shape[0]
        rope = self.ropes[l]
        ratio = cfg.ratio(l)
        kvv = self.pool.layer_views(l)
        ps = self.pool.page_size
        if yq is None:
            yq = O.fp8_quant(y)
        iw = None
        qkv = None
        if sp is not None:
            # the all-gather is fused into this GEMM's loads; everything else that reads y is issued behind it
            from ..ops.gemm import gemm_fp8_gated

            qkv = gemm_fp8_gated(yq[0], yq[1], w[p + "wqkv_a.weight"], w[p + "wqkv_a.scale"], sp[1])
        if ratio:
            # compressor (and indexer cache) branch: depends only on y, meets the query chain at the selection
            with self._fork(y):
                if ratio == 4:
                    iw = O.gemm_bf16(y, w[p + "idx.weights_proj"])
                    n1 = w[p + "comp.wkv_gate"].shape[0]
                    both = O.gemm_bf16(y, w[p + "comp_all.wkv_gate"], out_dtype=torch.float32)  # one GEMM, two slices
                    proj, proj_i = both[:, :n1], both[:, n1:]
                    pooled_i = O.compress(proj_i, fb, 4, cfg.index_head_dim, w[p + "idx.comp.ape"], kvv["idx_ring"],
                                          kvv["idx_ckpt"], ps)
                    O.indexer_kv_store(pooled_i, fb, w[p + "idx.comp.norm"], cfg.rms_norm_eps, rope, kvv["idx_vals"],
                                       kvv["idx_scale"], ps)
                else:
                    proj = O.gemm_bf16(y, w[p + "comp.wkv_gate"], out_dtype=torch.float32)
                pooled = O.compress(proj, fb, ratio, cfg.head_dim, w[p + "comp.ape"], kvv["ring"], kvv.get("ckpt"),
                                    ps)
                O.compress_store(pooled, fb, w[p + "comp.norm"], cfg.rms_norm_eps, rope, kvv["comp"], ps, ratio)
        if qkv is None:
            qkv = O.gemm_fp8(yq[0], yq[1], w[p + "wqkv_a.weight"], w[p + "wqkv_a.scale"])
        q_lora, qlq = O.rms_norm(qkv[:, : cfg.q_lora_rank], w[p + "q_norm.weight"], cfg.rms_norm_eps, want_q=True)
        kv = qkv[:, cfg.q_lora_rank:]
        q = O.gemm_fp8(qlq[0], qlq[1], w[p + "wq_b.weight"], w[p + "wq_b.scale"]).view(t, self.h_local, cfg.head_dim)
        q, kv = O.q_kv_norm_rope_store(q, kv, fb.positions, w[p + "kv_norm.weight"], cfg.rms_norm_eps, rope,
                                       kvv["swa"], fb.out_loc, self.pool.swa_map, ps, self.qat)
        topk_idx = topk_len = None
        if ratio == 4:
            iq = O.gemm_fp8(qlq[0], qlq[1], w[p + "idx.wq_b.weight"], w[p + "idx.wq_b.scale"])
            iq = iq.view(t, cfg.index_n_heads, cfg.index_head_dim)
        if ratio:
            self._join(y)
        if ratio == 4:
            qc, wf = O.indexer_q_encode(iq, iw, fb.positions, rope, cfg.index_head_dim ** -0.5,
                                        cfg.index_n_heads ** -0.5)
            topk_idx, topk_len = O.indexer_select(qc, wf, kvv["idx_vals"], kvv["idx_scale"], fb, ps, cfg.index_topk)
            if self._debug_bounds:
                O.check_index(topk_idx, -1, max(fb.max_context // 4, 1), "indexer_topk")
        o = O.attention(q, fb, kvv["swa"], self.pool.swa_map, kvv.get("comp"), ratio, topk_idx, topk_len,
                        w[p + "sink"], cfg.head_dim ** -0.5, ps, cfg.window_size, out_rope=rope)
        o2 = O.gemm_bf16_grouped(o.reshape(t, self.h_local * cfg.head_dim), w[p + "wo_a.weight_bf16"], self.g_local)
        if sp is not None:
            oq = O.fp8_quant(o2)
            self._mixed = True
            return self.comm.sp_gemm_fp8_reduce_scatter(sp[0], self.comm.CH_ATTN, oq[0], oq[1], w[p + "wo_b.weight"],
                                                        w[p + "wo_b.scale"], hc=hc)
        if getattr(self.comm, "fused", False):
            oq = O.fp8_quant(o2)
            self._mixed = hc is not None
            return self.comm.gemm_fp8_allreduce(oq[0], oq[1], w[p + "wo_b.weight"], w[p + "wo_b.scale"], hc=hc)
        out = self._fp8_linear(o2, p + "wo_b")
        return self.comm.all_reduce(out, "attn")

    def moe(self, l: int, y: torch.Tensor, fb: ForwardBatch, yq=None, hc=None, sp=None) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"L{l}.moe."
        if yq is None:
            yq = O.fp8_quant(y)
        gate_w = w[p + "gate.weight_bf16"] if y.is_cuda and (p + "gate.weight_bf16") in w else w[p + "gate.weight"]

        def shared_expert():
            with self._fork(y):  # beside the router / planning chain
                gu = O.gemm_fp8(yq[0], yq[1], w[p + "sh_gate_up.weight"], w[p + "sh_gate_up.scale"])
                aq = O.silu_mul_clamp_quant(gu, cfg.swiglu_limit)
                return O.gemm_fp8(aq[0], aq[1], w[p + "sh_down.weight"], w[p + "sh_down.scale"])

        def router(gate=None):
            return O.moe_gate(y, gate_w, w.get(p + "gate.bias"), cfg.num_experts_per_tok,
                              cfg.routed_scaling_factor, cfg.scoring_func, w.get(p + "gate.tid2eid"), fb.input_ids,
                              fb.num_valid, **({"gate": gate} if gate is not None else {}))

        if sp is not None:
            # row-sharded layer: the router GEMM's loads wait for the gathered rows; the shared expert follows it
            idx, wt = router(sp[1])
            shared = shared_expert()
        else:
            shared = shared_expert()
            idx, wt = router()
        if self._debug_bounds:
            O.check_index(idx, -1, cfg.n_routed_experts, "expert_ids")
        if y.is_cuda:
            # routed rows stay per route; the combine kernel sums them with the shared expert (and, with fused
            # communication, all-reduces the result in the same kernel)
            from ..ops import cuda as C

            rows, plan, mt = C.moe_routed(y, idx, wt, w[p + "w13"], w[p + "s13"], w[p + "w2"], w[p + "s2"],
                                          cfg.swiglu_limit, self.expert_base, cfg.n_routed_experts)
            t, k, h = y.shape[0], idx.shape[1], y.shape[1]
            self._join(y)
            if sp is not None:
                self._mixed = True
                return self.comm.sp_moe_finalize_reduce_scatter(sp[0], rows, plan, mt, shared, t, k, h, hc=hc)
            if getattr(self.comm, "fused", False):
                self._mixed = hc is not None
                return self.comm.moe_finalize_allreduce(rows, plan, mt, shared, fb.num_valid, t, k, h, hc=hc)
            if self.comm.size == 1:
                self._mixed = hc is not None
                return C.moe_finalize(rows, plan, mt, shared, fb.num_valid, t, k, h, hc)
            out = C.moe_finalize(rows, plan, mt, shared, fb.num_valid, t, k, h)
            return self.comm.all_reduce(out, "moe")
        routed = O.moe_experts(y, idx, wt, w[p + "w13"], w[p + "s13"], w[p + "w2"], w[p + "s2"], cfg.swiglu_limit,
                               self.expert_base)
        out = O.add_cast(routed, shared, fb.num_valid)
        return self.comm.all_reduce(out, "moe")

    def layer(self, l: int, x: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"L{l}."
        for blk, fn, norm in (("hc_attn", self.attention, "attn_norm"), ("hc_ffn", self.moe, "ffn_norm")):
            y, post, comb, yq = O.hc_pre(x, w[p + blk + ".fn"], w[p + blk + ".scale"], w[p + blk + ".base"],
                                         cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_norm_eps,
                                         w[p + norm + ".weight"], want_q=True)
            self._mixed = False
            y = fn(l, y, fb, yq, (x, post, comb))
            x = y if self._mixed else O.hc_post(y, x, post, comb)
        return x

    def layer_sp(self, l: int, x_own: torch.Tensor, fb: ForwardBatch, plan) -> torch.Tensor:
        """One layer with the residual streams sharded by rows (x_own = this rank's rows [n_own, 4, H]).  Per block:
        hyper-connection pre mix, norm and FP8 quantisation on the own rows only, written into the rank's rows of the
        gathered buffer; all-gather push; the block on all rows (heads / experts sharded as always), whose first GEMM
        consumes the gathered rows as they arrive and whose last kernel reduce-scatters; hyper-connection post mix
        on the own rows, fused behind the reduction."""
        cfg, w, p, c = self.cfg, self.w, f"L{l}.", self.comm
        t, r0, n = plan.t, plan.row0, plan.n_own
        for blk, fn, norm, ch in (("hc_attn", self.attention, "attn_norm", c.CH_ATTN),
                                  ("hc_ffn", self.moe, "ffn_norm", c.CH_MOE)):
            ag_y, ag_q, ag_s = c.sp_buffers(plan, ch)
            if n > 0:
                _, post, comb, _ = O.hc_pre(x_own, w[p + blk + ".fn"], w[p + blk + ".scale"], w[p + blk + ".base"],
                                            cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_norm_eps,
                                            w[p + norm + ".weight"], want_q=True,
                                            out=(ag_y[r0:r0 + n], ag_q[r0:r0 + n], ag_s[r0:r0 + n]))
            else:   # a short prompt leaves the last ranks without rows: they still take part in both exchanges
                post = torch.empty(0, cfg.hc_mult, dtype=torch.float32, device=x_own.device)
                comb = torch.empty(0, cfg.hc_mult, cfg.hc_mult, dtype=torch.float32, device=x_own.device)
            gate = c.sp_all_gather(plan, ch)
            x_own = fn(l, ag_y[:t], fb, (ag_q[:t], ag_s[:t]), (x_own, post, comb), sp=(plan, gate))
        return x_own

    def _forward_sp(self, fb: ForwardBatch, plan, greedy):
        cfg, w, c = self.cfg, self.w, self.comm
        r0, n = plan.row0, plan.n_own
        if n > 0:
            x_own = O.embed(fb.input_ids[r0:r0 + n], w["embed.weight"], cfg.hc_mult)
        else:
            x_own = torch.empty(0, cfg.hc_mult, cfg.hidden_size, dtype=w["embed.weight"].dtype,
                                device=fb.input_ids.device)
        for l in range(cfg.num_layers):
            x_own = self.layer_sp(l, x_own, fb, plan)
        # the rows whose logits are wanted live on their owners: every rank contributes its own ones, zeros elsewhere
        last = fb.last_idx if fb.last_idx is not None else torch.arange(plan.t, device=x_own.device)
        b, h = last.shape[0], cfg.hidden_size
        mine = (last >= r0) & (last < r0 + n)
        sel = torch.zeros(b, cfg.hc_mult, h, dtype=x_own.dtype, device=x_own.device)
        if n > 0:
            sel[mine] = x_own[(last[mine] - r0)]
        x = c.all_reduce(sel.view(b * cfg.hc_mult, h)).view(b, cfg.hc_mult, h)
        y = O.hc_head(x, w["hc_head.fn"], w["hc_head.scale"], w["hc_head.base"], cfg.hc_eps, cfg.rms_norm_eps,
                      w["norm.weight"])
        logits = O.gemm_bf16(y, w["head.weight"], out_dtype=torch.float32)
        if greedy is not None:
            return logits, c.greedy_tokens(logits, fb.slots[last], None, greedy)
        return c.all_gather_last(logits)

    # ------------------------------------------------------------------ forward
    def prepare_report(self) -> dict:
        """What the loaded weights occupy on this rank, by storage format, and which derived tensors were built at
        load time.  The reference rebuilds BF16 caches and a Marlin repack at every start and reports them in
        ``model_prepare_report`` (python/minisgl/models/deepseek_v4.py:1718-1787); here the FP8 projections are
        consumed in place and the FP4 experts are only re-ordered (same bytes), so the derived part is small: the
        dequantised ``wo_a``, the bf16 router weight and the stacked compressor projection."""
        by_fmt, derived = {}, {}
        for k, v in self.w.items():
            if not isinstance(v, torch.Tensor):
                continue
            n = v.numel() * v.element_size()
            if k.endswith((".w13", ".w2")):
                fmt = "fp4_packed"
            elif k.endswith((".s13", ".s2")):
                fmt = "e8m0_scales"
            else:
                fmt = str(v.dtype).replace("torch.", "")
            by_fmt[fmt] = by_fmt.get(fmt, 0) + n
            if k.endswith(("gate.weight_bf16", "comp_all.wkv_gate")) or ".wo_a." in k and v.dtype == torch.bfloat16:
                derived[k.split(".", 1)[1]] = derived.get(k.split(".", 1)[1], 0) + n
        return {"rank": self.comm.rank, "world": self.comm.size, "moe_mode": self.moe_mode,
                "experts_local": int(self.w["L0.moe.w13"].shape[0]), "expert_base": self.expert_base,
                "heads_local": self.h_local, "o_groups_local": self.g_local,
                "bytes_by_format": by_fmt, "bytes_total": sum(by_fmt.values()),
                "derived_bytes": derived, "repack": "experts re-tiled in place for the block-scaled GEMM (same bytes); FP8 projections read in place",
                "weight_prefetch_before_dependency_wait": bool(self.w["embed.weight"].is_cuda)}

    def audit_inputs(self, fb: ForwardBatch) -> None:
        """Checked runs (MINISGL_DEBUG_BOUNDS=1): every index tensor the kernels gather with is audited against its
        range before use; a violation is recorded in the device status word (CPU: raised) instead of being
        dereferenced.  The sanitizer-free counterpart of the reference's fail-closed wrappers
        (python/minisgl/kernel/deepseek_v4.py of the reference validates shapes and dtypes, not values)."""
        cfg = self.cfg
        locs = self.pool.sizes.num_pages * self.pool.page_size
        O.check_index(fb.input_ids, 0, cfg.vocab_size, "input_ids")
        O.check_index(fb.positions, 0, fb.page_table.shape[1], "positions")
        O.check_index(fb.slots, 0, fb.page_table.shape[0], "slots")
        O.check_index(fb.out_loc, -1, locs, "out_loc")
        O.check_index(fb.page_table, 0, locs, "page_table")

    def forward(self, fb: ForwardBatch, greedy: Optional[GreedyTail] = None):
        """Returns fp32 logits [B, vocab] for the rows ``fb.last_idx``; with ``greedy`` returns
        (this rank's logits shard [B, vocab / tp], greedy tokens [B] int32) and skips the logits all-gather."""
        cfg, w = self.cfg, self.w
        if self._debug_bounds and fb.token_feedback is None:
            self.audit_inputs(fb)
        if fb.is_prefill and fb.input_ids.is_cuda and hasattr(self.comm, "sp_plan") and self.moe_mode == "ep":
            plan = self.comm.sp_plan(fb.input_ids.shape[0])
            if plan is not None:
                return self._forward_sp(fb, plan, greedy)
        x = O.embed(fb.input_ids, w["embed.weight"], cfg.hc_mult, fb.token_feedback,
                    fb.slots if fb.token_feedback is not None else None)
        if self._debug_bounds and fb.token_feedback is not None:
            self.audit_inputs(fb)
        for l in range(cfg.num_layers):
            x = self.layer(l, x, fb)
        if fb.last_idx is not None and (fb.is_prefill or fb.last_idx.shape[0] != x.shape[0]):
            x = x[fb.last_idx].contiguous()
        y = O.hc_head(x, w["hc_head.fn"], w["hc_head.scale"], w["hc_head.base"], cfg.hc_eps, cfg.rms_norm_eps,
                      w["norm.weight"])
        if greedy is not None and greedy.logits_out is not None:
            logits = O.gemm_bf16(y, w["head.weight"], out=greedy.logits_out[: y.shape[0]])
        else:
            logits = O.gemm_bf16(y, w["head.weight"], out_dtype=torch.float32)
        if greedy is not None:
            gathered = fb.last_idx is not None and (fb.is_prefill or fb.last_idx.shape[0] != fb.slots.shape[0])
            slots = fb.slots[fb.last_idx] if gathered else fb.slots
            return logits, self.comm.greedy_tokens(logits, slots, None if gathered else fb.num_valid, greedy)
        return self.comm.all_gather_last(logits)
