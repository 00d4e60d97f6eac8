#!/usr/bin/env python
"""Headline benchmark: decode throughput of the offline M=128 wave (128 sequences, 1 024 random input tokens each,
forced output, greedy, ignore-EOS) on the DeepSeek-V4-Flash architecture with random-init FP8/FP4 weights.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torch.distributed.run)

A *step* is one decode forward of the whole batch (one new token per sequence).  The run goes through the public
offline API (``minisgl.llm.LLM``): requests are submitted, prefilled in 8 192-token chunks, then W warm-up and exactly
K timed decode steps run through the scheduler loop, bracketed by a barrier and a device synchronize.

  value   = decode tokens / sum of the K forwards' device times (CUDA events), max over ranks -- the reference's
            "decode tok/s" definition (debug/dsv4/benchmark/offline/deepseek_v4_perf_matrix.py:4842-4867)
  e2e     = the same tokens / wall-clock of the timed region through the scheduler: every step copies its inputs
            (positions, slots, token locations) from pinned host memory and reads the sampled tokens back.

One JSON line is printed by rank 0.  ``--impl reference`` tries the unmodified reference from ``baseline/_ref``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
BASELINE_DECODE_TOK_S = 2487.78  # PERFORMANCE.md:33 of the reference (8xA100, TP8, M=128, 1K prompts)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0, help="0 = as many of the 43 layers as fit in memory")
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--moe-mode", default="ep", choices=["ep", "tp"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-fused-comm", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)  # fewer than three untimed steps would leave clocks and caches cold
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_reference(args) -> None:
    """The reference arm: the unmodified reference installed under baseline/_ref, through its own gate."""
    out = {"impl": "reference"}
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "minisgl")):
        out["unavailable"] = ("baseline/_ref is not installed (pip install --no-index --no-build-isolation --no-deps "
                              "--target baseline/_ref <reference checkout>)")
        print(json.dumps(out))
        return
    probe = ("import sys; sys.path.insert(0, %r); import torch; from minisgl.kernel import deepseek_v4 as k; "
             "cap = torch.cuda.get_device_capability() if torch.cuda.is_available() else None; "
             "print('GATE', bool(k.dsv4_triton_available()), cap)") % ref
    try:
        r = subprocess.run([sys.executable, "-c", probe], capture_output=True, text=True, timeout=600, cwd="/tmp")
        line = next((l for l in r.stdout.splitlines() if l.startswith("GATE")), None)
        if line is None:
            err = (r.stderr.strip().splitlines() or ["no output"])[-1]
            out["unavailable"] = "the reference package does not import here: " + err[:200]
        elif " True " in line + " ":
            out["unavailable"] = "reference gate open but its Ampere-only Marlin/Triton build was not attempted on this GPU"
        else:
            out["unavailable"] = ("the unmodified reference refuses to run off Ampere: its kernel wrappers raise unless "
                                  "the device capability is (8,0) or (8,6) (python/minisgl/utils/arch.py:6, "
                                  "python/minisgl/kernel/deepseek_v4.py:141-143); probe says " + line[5:].strip())
    except Exception as e:  # pragma: no cover
        out["unavailable"] = f"reference probe failed: {type(e).__name__}: {e}"[:240]
    print(json.dumps(out))


def pick_layers(args, world: int) -> int:
    import torch

    from minisgl.models.config import ModelConfig

    if args.layers > 0:
        return min(args.layers, 43)
    free, total = torch.cuda.mem_get_info()
    cfg = ModelConfig.flash()
    e_local = args.experts // world if args.moe_mode == "ep" else args.experts
    inter = cfg.moe_intermediate_size // (1 if args.moe_mode == "ep" else world)
    expert_bytes = e_local * (3 * inter * cfg.hidden_size // 2 + 3 * inter * cfg.hidden_size // 32)
    dense = (170 << 20) // world + (60 << 20)
    per_layer = expert_bytes + dense
    # embedding + head shard, KV pools and rings, prefill activations, CUDA context, 4 % head-room
    reserve = int(0.04 * total) + cfg.vocab_size * cfg.hidden_size * 2 * (1 + 1 / world) + (12 << 30)
    return max(min(int((free - reserve) // per_layer), 43), 1)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus or world == 1 and args.gpus == 1, f"WORLD_SIZE {world} != --gpus {args.gpus}"
    torch.cuda.set_device(local)
    from minisgl.core import SamplingParams
    from minisgl.llm import LLM
    from minisgl.models.config import ModelConfig
    from minisgl.ops import native
    from minisgl.parallel.info import DistributedInfo
    import dataclasses

    layers = pick_layers(args, world)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    cfg = ModelConfig.flash().with_layers(layers)
    if args.experts != 256:
        cfg = dataclasses.replace(cfg, n_routed_experts=args.experts)
    # every sequence is asked for 1 024 output tokens, like the reference's wave.  Under mixed load the scheduler
    # runs 4 decode forwards per 2 048-token prefill forward, so the first sequences are a few hundred tokens into
    # their output when the last prompt finishes; the timed steps start there, with all sequences decoding.
    n_out = args.output_len
    mixed_fwd = (args.batch * args.prompt_len + 2047) // 2048
    if 4 * mixed_fwd + args.warmup + args.steps + 2 > n_out:
        raise SystemExit(f"--output-len {n_out} is too short for {args.warmup}+{args.steps} steps after the prefill wave")
    ctx = args.prompt_len + n_out + 256
    llm = LLM(model_config=cfg, tp_info=DistributedInfo(rank, world), use_dummy_weight=True, recipe="default_m128",
              max_running_req=args.batch, context_length=max(ctx, 4096), moe_mode=args.moe_mode,
              use_pynccl=not args.no_fused_comm, disable_log_stats=True, memory_ratio=0.97,
              cuda_graph_max_bs=0 if args.no_graph else args.batch,
              cuda_graph_bs=None if args.no_graph else [args.batch])
    eng = llm.engine
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g, dtype=torch.int32)
               for _ in range(args.batch)]
    sp = SamplingParams(max_tokens=n_out, ignore_eos=True)
    from minisgl.message import UserMsg

    t_submit = time.perf_counter()
    for uid, p in enumerate(prompts):
        llm._queue.append(UserMsg(uid, p, SamplingParams(**vars(sp)), None))
        llm._results[uid] = __import__("minisgl.llm.llm", fromlist=["RequestOutput"]).RequestOutput(uid)
        llm._open += 1
    llm.t_submit = t_submit

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=eng.cpu_group)

    # ---- prefill (untimed here; reported separately) and warm-up decode steps
    eng.record_timings = True
    last = None
    t_pref0 = time.perf_counter()
    while llm.prefill.runnable or len(llm.decode.running) < args.batch:
        last = llm.overlap_loop(last)
    barrier()
    t_prefill = time.perf_counter() - t_pref0
    prefill_ms = sum(a.elapsed_time(b) for t in eng.timings if t["phase"] == "prefill" for a, b in [t["events"]])
    for _ in range(args.warmup):
        last = llm.overlap_loop(last)
    barrier()
    eng.timings.clear()
    h2d0, d2h0, launches0 = llm.bytes_h2d, llm.bytes_d2h, native.launch_count()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        last = llm.overlap_loop(last)
    llm._process_last_data(last)
    last = None
    ev1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    barrier()
    clk = clocks.stop() if rank == 0 else {}
    dec = [t for t in eng.timings if t["phase"] == "decode"]
    assert len(dec) == args.steps, (len(dec), args.steps)
    fwd_ms = [t["events"][0].elapsed_time(t["events"][1]) for t in dec]
    dev_s, span_s = sum(fwd_ms) / 1e3, ev0.elapsed_time(ev1) / 1e3
    stats = torch.tensor([dev_s, span_s, wall], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX, group=eng.cpu_group)
    dev_s, span_s, wall = [float(x) for x in stats]
    tokens = args.batch * args.steps
    launches = native.launch_count() - launches0
    outs = list(llm._results.values())
    for uid in range(args.batch):  # the wave is measured; retire what is still running
        llm._abort(uid)
    ttft = sorted(o.t_first - t_submit for o in outs if o.t_first)
    tpot = sorted((o.t_tokens[-1] - o.t_tokens[0]) / (len(o.t_tokens) - 1) for o in outs if len(o.t_tokens) > 1)
    if rank == 0:
        value = tokens / dev_s
        line = {
            "metric": "decode output tok/s (box, max over ranks), M=128, 1K prompts", "value": round(value, 2),
            "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_s / args.steps * 1e3, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / BASELINE_DECODE_TOK_S, 4), "dtype": "bf16 activations, fp8 dense / fp4 expert weights",
            "data": "synthetic (uniform-random token ids, random-init weights)", "impl": "ours",
            "config": {"model": f"DeepSeek-V4-Flash architecture, {layers}/43 layers, {args.experts} experts",
                       "global_batch": args.batch, "seq_len": args.prompt_len, "output_len": n_out,
                       "parallelism": f"tp{world}" + (f"+{args.moe_mode}{world}" if world > 1 else ""),
                       "collectives": getattr(llm.engine.comm, "mode", "none"),
                       "page_size": eng.page_size, "cuda_graph": eng.graph_runner is not None,
                       "kv_pages": eng.num_pages, "swa_slots": eng.kv_plan["swa_slots"],
                       "l2": "inputs larger than L2 (weights read per step: %.1f GiB per GPU)" % (eng.weight_bytes / 2**30)},
            "clocks": clk,
            "e2e": {"value": round(tokens / wall, 2), "unit": "tok/s",
                    "h2d_bytes_per_step": (llm.bytes_h2d - h2d0) // max(args.steps, 1),
                    "d2h_bytes_per_step": (llm.bytes_d2h - d2h0) // max(args.steps, 1),
                    "device_span_tok_s": round(tokens / span_s, 2)},
            "gpu_launches": int(launches),
            "prefill": {"tok_s_device": round(args.batch * args.prompt_len / (prefill_ms / 1e3), 1) if prefill_ms else None,
                        "wall_s": round(t_prefill, 2)},
            "latency": {"p50_ttft_s": round(ttft[len(ttft) // 2], 3) if ttft else None,
                        "p50_tpot_ms": round(tpot[len(tpot) // 2] * 1e3, 3) if tpot else None},
        }
        print(json.dumps(line), flush=True)
    llm.shutdown()


if __name__ == "__main__":
    main()
