"""No-weight simulation of the scheduler's policies: the real ``MixedPhaseFairPolicy`` and
``allocate_fair_prefill_chunks`` drive a toy engine whose forward costs come from a linear cost model, so phase
arbitration and long-prefill fairness can be studied in milliseconds on a CPU (the reference ships such harnesses
under benchmark/scheduler_*; this is the same idea on this engine's policy code).

    python -m minisgl.benchmark.scheduler_sim --scenario long_prefill
    python -m minisgl.benchmark.scheduler_sim --scenario mixed --decode-first 1 --max-consecutive-decode 4

Prints a JSON summary: per-request TTFT, decode stall statistics (gaps between decode steps while prefills run),
and, for fairness, the step at which each prompt finished its prefill.
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass, field
from typing import List

from minisgl.scheduler.phase_policy import MixedPhaseFairPolicy
from minisgl.scheduler.prefill import allocate_fair_prefill_chunks


@dataclass
class SimReq:
    uid: int
    arrival_ms: float
    prompt: int
    output: int
    done_prefill: int = 0
    granted: int = 0
    generated: int = 0
    t_first: float = -1.0
    t_done: float = -1.0
    prefill_done_step: int = -1
    token_times: List[float] = field(default_factory=list)


def cost_prefill_ms(tokens: int) -> float:
    return 1.5 + tokens * 0.0045        # ~8192 tokens in ~38 ms


def cost_decode_ms(batch: int) -> float:
    return 6.0 + batch * 0.05           # ~12 ms at batch 128


def simulate(reqs: List[SimReq], *, budget: int = 8192, mixed_budget: int = 2048, max_consecutive_decode: int = 4,
             first_conflict: str = "decode", page: int = 256, max_running: int = 256) -> dict:
    policy = MixedPhaseFairPolicy(isolated_prefill_budget=budget, mixed_prefill_budget=mixed_budget,
                                  max_consecutive_decode=max_consecutive_decode, first_conflict=first_conflict)
    now, step = 0.0, 0
    pending = sorted(reqs, key=lambda r: r.arrival_ms)
    resident: List[SimReq] = []
    running: List[SimReq] = []
    finished: List[SimReq] = []
    trace = []
    while pending or resident or running:
        arrived = [r for r in pending if r.arrival_ms <= now]
        while arrived and len(resident) + len(running) < max_running:
            r = arrived.pop(0)
            pending.remove(r)
            resident.append(r)
        pre, dec = bool(resident), bool(running)
        d = policy.choose(prefill_runnable=pre, decode_runnable=dec)
        if d.phase is None:
            now = pending[0].arrival_ms  # idle until the next arrival
            policy.record_scheduled(None, prefill_runnable=False, decode_runnable=False)
            continue
        if d.phase == "prefill":
            q = min(page, d.prefill_budget)
            chosen = resident[: max(d.prefill_budget // q, 1)]
            grants = allocate_fair_prefill_chunks(token_budget=d.prefill_budget, alignment_quantum=q,
                                                  scheduled_tokens=[r.granted for r in chosen],
                                                  remaining_tokens=[r.prompt - r.done_prefill for r in chosen])
            now += cost_prefill_ms(sum(grants))
            ran = []
            for r, g in zip(chosen, grants):
                if g <= 0:
                    continue
                r.done_prefill += g
                r.granted += g
                ran.append(r)
                if r.done_prefill >= r.prompt:
                    r.t_first, r.prefill_done_step = now, step
                    r.generated = 1
                    r.token_times.append(now)
                    resident.remove(r)
                    (finished if r.generated >= r.output else running).append(r)
                    if r.generated >= r.output:
                        r.t_done = now
            resident = [r for r in resident if r not in ran] + [r for r in resident if r in ran]
            trace.append(("P", sum(grants)))
        else:
            now += cost_decode_ms(len(running))
            for r in list(running):
                r.generated += 1
                r.token_times.append(now)
                if r.generated >= r.output:
                    r.t_done = now
                    running.remove(r)
                    finished.append(r)
            trace.append(("D", len(running)))
        policy.record_scheduled(d.phase, prefill_runnable=pre, decode_runnable=dec)
        step += 1
    gaps = []
    for r in finished:
        gaps += [b - a for a, b in zip(r.token_times, r.token_times[1:])]
    gaps.sort()
    ttft = sorted(r.t_first - r.arrival_ms for r in finished)

    def pct(xs, q):
        return xs[min(int(q * (len(xs) - 1) + 0.5), len(xs) - 1)] if xs else None

    return {
        "steps": step, "makespan_ms": round(now, 2), "prefill_steps": sum(1 for t in trace if t[0] == "P"),
        "decode_steps": sum(1 for t in trace if t[0] == "D"),
        "ttft_ms": {"p50": pct(ttft, 0.5), "p99": pct(ttft, 0.99), "max": ttft[-1] if ttft else None},
        "inter_token_ms": {"p50": pct(gaps, 0.5), "p99": pct(gaps, 0.99), "max": gaps[-1] if gaps else None},
        "prefill_done_step": {r.uid: r.prefill_done_step for r in sorted(finished, key=lambda r: r.uid)[:16]},
        "first_steps": "".join(t[0] for t in trace[:64]),
    }


def scenario(name: str) -> List[SimReq]:
    if name == "long_prefill":      # one 64 K prompt and 15 short ones arrive together
        return [SimReq(0, 0.0, 65536, 32)] + [SimReq(i, 0.0, 512, 32) for i in range(1, 16)]
    if name == "mixed":             # 64 decoding requests, a new 4 K prompt every 50 ms
        return [SimReq(i, 0.0, 256, 256) for i in range(64)] + [SimReq(64 + i, 50.0 * (i + 1), 4096, 64)
                                                               for i in range(16)]
    if name == "wave":              # the benchmark wave: 128 x 1 K prompts, 1 K outputs
        return [SimReq(i, 0.0, 1024, 1024) for i in range(128)]
    raise SystemExit(f"unknown scenario {name!r}; choose long_prefill, mixed or wave")


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenario", default="mixed")
    ap.add_argument("--budget", type=int, default=8192)
    ap.add_argument("--mixed-budget", type=int, default=2048)
    ap.add_argument("--max-consecutive-decode", type=int, default=4)
    ap.add_argument("--decode-first", type=int, default=1)
    a = ap.parse_args(argv)
    res = simulate(scenario(a.scenario), budget=a.budget, mixed_budget=a.mixed_budget,
                   max_consecutive_decode=a.max_consecutive_decode,
                   first_conflict="decode" if a.decode_first else "prefill")
    res["scenario"] = a.scenario
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
