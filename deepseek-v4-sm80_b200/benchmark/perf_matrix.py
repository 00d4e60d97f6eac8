"""Scenario matrix over the offline engine: the same catalogue the reference's perf-matrix harness runs
(benchmark/perf_matrix: P1K / P4K prompts x M concurrent requests, mixed arrival, one long resident prompt beside
short ones, KV-pressure cases), each scenario through an instrumented ``LLM`` that records per-request TTFT / TPOT,
engine step counts per phase and prefix-cache metrics.

    python -m minisgl.benchmark.perf_matrix --dummy --layers 4 --scenarios P1K_M32 P1K_M128 MIXED_ARRIVAL

With ``--dummy`` the model is random-init (``--layers`` trims its depth so that it fits a small GPU or a CPU run with
the tiny config, ``--tiny``).  Prints one JSON object per scenario and a final summary list.

Instrumentation (the reference's harness records the same things,
debug/dsv4/benchmark/offline/deepseek_v4_perf_matrix.py:2836-2970, :3096-3140, :4842-4867):
  * ``--timings``        device time of every forward (CUDA events around ``Engine.forward_batch``), summed per phase:
                         prefill tok/s = prompt tokens / sum of prefill-forward seconds, decode tok/s likewise, plus
                         the host time the scheduler spent preparing batches (wall minus device)
  * ``--ledger``         memory ledger: weights, KV plan, CUDA-graph pool, allocator peak, free device memory
  * ``--trace-kernels``  per native launcher: calls and device milliseconds (events around every launch; slows the run,
                         so its throughput figures are not benchmark numbers)
Long-context entries (LONG_128K, LONG_512K_M8, LONG_1M_M4) follow the reference's capability smokes
(PERFORMANCE.md:61-62): prompts that differ at token 0, a few decode tokens, chunked prefill at the 8 192 budget.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
from dataclasses import dataclass
from typing import Dict, List


@dataclass(frozen=True)
class Scenario:
    name: str
    prompt_lens: tuple          # one entry per request
    output_len: int
    arrival_gap_steps: int = 0  # 0: all requests present at the start; k: one new request every k engine steps
    note: str = ""


def catalogue(scale: float = 1.0) -> Dict[str, Scenario]:
    def n(x):
        return max(int(x * scale), 1)

    c = {}
    for p, tag in ((1024, "P1K"), (4096, "P4K")):
        for m in (1, 8, 32, 64, 128, 256):
            c[f"{tag}_M{m}"] = Scenario(f"{tag}_M{m}", (n(p),) * m, n(256), note="uniform wave")
    c["MIXED_ARRIVAL"] = Scenario("MIXED_ARRIVAL", tuple(n(x) for x in (1024, 256, 4096, 512) * 16), n(128), 2,
                                  "requests trickle in while others decode: exercises the mixed-phase policy")
    c["LONG_RESIDENT_64K"] = Scenario("LONG_RESIDENT_64K", (n(65536),) + (n(512),) * 31, n(128), 0,
                                      "one 64 K prompt beside 31 short ones: fair chunked prefill must not starve them")
    c["PRESSURE_512K"] = Scenario("PRESSURE_512K", (n(8192),) * 64, n(256), 0, "512 Ki resident tokens")
    c["PRESSURE_1M"] = Scenario("PRESSURE_1M", (n(16384),) * 64, n(256), 0, "1 Mi resident tokens: admission waits")
    c["LONG_128K"] = Scenario("LONG_128K", (n(131072),), 16, 0, "one 128 Ki prompt + 16 decode tokens")
    c["LONG_512K_M8"] = Scenario("LONG_512K_M8", (n(524288),) * 8, 8, 0, "eight 512 Ki prompts + 8 decode tokens")
    c["LONG_1M_M4"] = Scenario("LONG_1M_M4", (n(1048576 - 8),) * 4, 8, 0, "four sequences of 1 Mi total tokens")
    c["SHARED_PREFIX"] = Scenario("SHARED_PREFIX", (n(2048),) * 32, n(64), 4,
                                  "identical prompts arriving over time: radix prefix hits")
    return c


def _percentile(xs: List[float], q: float) -> float:
    if not xs:
        return float("nan")
    xs = sorted(xs)
    return xs[min(int(q * (len(xs) - 1) + 0.5), len(xs) - 1)]


def run_scenario(llm, sc: Scenario, seed: int = 0) -> dict:
    import torch

    from minisgl.core import SamplingParams

    vocab = llm.engine.model_config.vocab_size
    g = torch.Generator().manual_seed(seed)
    if sc.name == "SHARED_PREFIX":
        base = torch.randint(0, vocab, (sc.prompt_lens[0],), generator=g, dtype=torch.int32)
        prompts = [base.clone() for _ in sc.prompt_lens]
    else:
        prompts = [torch.randint(0, vocab, (p,), generator=g, dtype=torch.int32) for p in sc.prompt_lens]
    steps0 = dict(getattr(llm, "phase_steps", {}))
    eng = llm.engine
    eng.timings = []
    if eng.is_cuda:
        torch.cuda.reset_peak_memory_stats(eng.device)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, SamplingParams(max_tokens=sc.output_len, ignore_eos=True),
                        arrival_gap_steps=sc.arrival_gap_steps)
    wall = time.perf_counter() - t0
    ttft = [o.t_first - t0 for o in outs if o.t_first is not None]
    tpot = []
    for o in outs:
        if len(o.t_tokens) > 1:
            tpot.append((o.t_tokens[-1] - o.t_tokens[0]) / (len(o.t_tokens) - 1))
    n_out = sum(len(o.token_ids) for o in outs)
    steps1 = dict(getattr(llm, "phase_steps", {}))
    extra = {}
    if eng.record_timings and eng.timings:
        torch.cuda.synchronize(eng.device)
        per = {"prefill": [0.0, 0, 0], "decode": [0.0, 0, 0]}
        for t in eng.timings:
            ms = t["events"][0].elapsed_time(t["events"][1])
            per[t["phase"]][0] += ms
            per[t["phase"]][1] += t["tokens"]
            per[t["phase"]][2] += 1
        dev_s = (per["prefill"][0] + per["decode"][0]) / 1e3
        extra["forwards"] = {
            ph: {"count": v[2], "tokens": v[1], "device_s": round(v[0] / 1e3, 4),
                 "tok_s": round(v[1] / (v[0] / 1e3), 1) if v[0] > 0 else None,
                 "ms_per_forward": round(v[0] / v[2], 3) if v[2] else None} for ph, v in per.items()}
        extra["host_s_outside_forwards"] = round(wall - dev_s, 4)
    if eng.is_cuda:
        extra["peak_allocated_gib"] = round(torch.cuda.max_memory_allocated(eng.device) / 2**30, 3)
    return {**extra,
        "scenario": sc.name, "note": sc.note, "requests": len(outs), "prompt_tokens": int(sum(sc.prompt_lens)),
        "output_tokens": n_out, "wall_s": round(wall, 4), "output_tok_s": round(n_out / wall, 2),
        "ttft_s": {"p50": _percentile(ttft, 0.5), "p99": _percentile(ttft, 0.99), "max": max(ttft) if ttft else None},
        "tpot_ms": {"p50": 1e3 * _percentile(tpot, 0.5), "p99": 1e3 * _percentile(tpot, 0.99),
                    "mean": 1e3 * statistics.fmean(tpot) if tpot else None},
        "steps": {k: steps1.get(k, 0) - steps0.get(k, 0) for k in steps1},
        "prefix": llm.cache.prefix_metrics_snapshot(),
    }


def main(argv=None) -> List[dict]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--tiny", action="store_true", help="tiny architecture (CPU-sized); implies --dummy")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--scale", type=float, default=1.0, help="multiplies every length of the catalogue")
    ap.add_argument("--max-running", type=int, default=256)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--page-size", type=int, default=256)
    ap.add_argument("--num-pages", type=int, default=0, help="override the KV page count (CPU runs need it)")
    ap.add_argument("--scenarios", nargs="*", default=["P1K_M32", "P1K_M128", "MIXED_ARRIVAL"])
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--timings", action="store_true", help="device time per forward, per-phase tok/s")
    ap.add_argument("--ledger", action="store_true", help="memory ledger after start-up and after the run")
    ap.add_argument("--trace-kernels", action="store_true", help="per-launcher call counts and device time")
    ap.add_argument("--experts", type=int, default=0, help="routed experts of the random-init model (0: the full 256)")
    ap.add_argument("--graph-bs", type=int, nargs="*", default=None, help="CUDA-graph batch sizes (default: recipe)")
    ap.add_argument("--recipe", default="", help="serving recipe (sets max running requests and graph buckets)")
    a = ap.parse_args(argv)
    cat = catalogue(a.scale)
    if a.list:
        for s in cat.values():
            print(f"{s.name:20s} requests={len(s.prompt_lens):4d} prompt={max(s.prompt_lens):6d} out={s.output_len} {s.note}")
        return []
    from minisgl.llm import LLM
    from minisgl.models.config import ModelConfig

    kw = {}
    if a.tiny or a.dummy or not a.model:
        import dataclasses

        cfg = ModelConfig.tiny() if a.tiny else ModelConfig.flash()
        cfg = cfg.with_layers(a.layers) if a.layers else cfg
        if a.experts:
            cfg = dataclasses.replace(cfg, n_routed_experts=a.experts)
        kw = dict(model_config=cfg, use_dummy_weight=True)
    if a.graph_bs is not None:
        kw["cuda_graph_bs"] = a.graph_bs
    longest = max(max(cat[s].prompt_lens) + cat[s].output_len for s in a.scenarios)
    if a.num_pages:
        kw["num_page_override"] = a.num_pages
    if a.recipe:
        kw["recipe"] = a.recipe
    else:
        kw["max_running_req"] = a.max_running
    t_start = time.perf_counter()
    llm = LLM(a.model, context_length=max(longest + 64, 4096), device=a.device, page_size=a.page_size, **kw)
    if llm.tp.is_primary():
        gr = llm.engine.graph_runner
        print(json.dumps({"startup_s": round(time.perf_counter() - t_start, 2),
                          "graphs_captured": gr.capture_status["captured"] if gr is not None else 0,
                          "graph_buckets": gr.buckets if gr is not None else [],
                          "context_classes": gr.classes if gr is not None else []}), flush=True)
    llm.engine.record_timings = bool(a.timings) and llm.engine.is_cuda
    if a.trace_kernels and llm.engine.is_cuda:
        from minisgl.ops import native

        native.enable_profile(True)
    if a.ledger and llm.tp.is_primary():
        print(json.dumps({"ledger": memory_ledger(llm), "when": "after start-up"}), flush=True)
    results = []
    for name in a.scenarios:
        res = run_scenario(llm, cat[name])
        if a.trace_kernels and llm.engine.is_cuda:
            from minisgl.ops import native

            res["kernels"] = {k: {"calls": c, "ms": round(ms, 3)} for k, (c, ms) in native.profile_report().items()}
        if a.ledger:
            res["ledger"] = memory_ledger(llm)
        results.append(res)
        if llm.tp.is_primary():
            print(json.dumps(res), flush=True)
    llm.shutdown()
    return results


def memory_ledger(llm) -> dict:
    """Where the device memory went: weights, the KV plan (pages, window slots, request slots), the captured graphs'
    pool against its estimate, the allocator's current / peak figures and what the device still has free."""
    import torch

    eng = llm.engine
    out = {"weights_gib": round(eng.weight_bytes / 2**30, 3), "kv_plan": dict(eng.kv_capacity_plan_report),
           "graphs": getattr(eng, "graph_memory_report", None),
           "graph_launches": dict((f"{k[0]}x{k[1]}", v) for k, v in eng.graph_runner.launches.items())
           if eng.graph_runner is not None else None}
    if eng.is_cuda:
        free, total = torch.cuda.mem_get_info(eng.device)
        out.update({"allocated_gib": round(torch.cuda.memory_allocated(eng.device) / 2**30, 3),
                    "reserved_gib": round(torch.cuda.memory_reserved(eng.device) / 2**30, 3),
                    "peak_allocated_gib": round(torch.cuda.max_memory_allocated(eng.device) / 2**30, 3),
                    "device_free_gib": round(free / 2**30, 3), "device_total_gib": round(total / 2**30, 3)})
    g = out["graphs"]
    if g is not None and not isinstance(g, dict):
        out["graphs"] = dict(vars(g)) if hasattr(g, "__dict__") else str(g)
    return out


if __name__ == "__main__":
    main()
