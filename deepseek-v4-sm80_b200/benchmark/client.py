"""Async load generator for the OpenAI-compatible server and its latency statistics.

``benchmark_trace`` replays a list of ``TraceItem`` (arrival time, prompt, output length) against
``/v1/chat/completions`` with streaming, records a timestamp per received chunk and reports TTFT / TPOT / E2E
(avg, p50, p90, p99, max) and throughput.  ``synthetic_chat_trace`` builds the online workload used here: Poisson
arrivals, log-normal prompt / output lengths, a fraction of requests sharing a common prefix (exercises the radix
cache).  ``read_qwen_trace`` / ``read_mooncake_trace`` parse the public trace formats; ``scale_traces`` compresses
or stretches arrival times.  Counterpart of python/minisgl/benchmark/client.py:18-498 of the reference.
"""
from __future__ import annotations

import asyncio
import json
import math
import random
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence


@dataclass
class TraceItem:
    arrival_s: float
    prompt: str
    output_len: int
    input_len: int = 0


@dataclass
class RequestResult:
    tics: List[float] = field(default_factory=list)   # time of every streamed chunk
    t_start: float = 0.0
    ok: bool = True
    output_tokens: int = 0

    @property
    def ttft(self) -> Optional[float]:
        return self.tics[0] - self.t_start if self.tics else None

    @property
    def tpot(self) -> Optional[float]:
        return (self.tics[-1] - self.tics[0]) / (len(self.tics) - 1) if len(self.tics) > 1 else None

    @property
    def e2e(self) -> Optional[float]:
        return self.tics[-1] - self.t_start if self.tics else None


def percentile(xs: Sequence[float], p: float) -> float:
    xs = sorted(xs)
    if not xs:
        return float("nan")
    k = (len(xs) - 1) * p / 100.0
    lo, hi = math.floor(k), math.ceil(k)
    return xs[lo] if lo == hi else xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def summarize(results: Sequence[RequestResult], wall_s: float) -> Dict[str, Any]:
    out: Dict[str, Any] = {"requests": len(results), "failed": sum(not r.ok for r in results), "wall_s": wall_s}
    for name in ("ttft", "tpot", "e2e"):
        xs = [getattr(r, name) for r in results if r.ok and getattr(r, name) is not None]
        out[name] = {"avg": sum(xs) / len(xs) if xs else float("nan"), "p50": percentile(xs, 50),
                     "p90": percentile(xs, 90), "p99": percentile(xs, 99), "max": max(xs) if xs else float("nan")}
    toks = sum(len(r.tics) for r in results if r.ok)
    out["output_tok_s"] = toks / wall_s if wall_s > 0 else float("nan")
    out["req_s"] = sum(r.ok for r in results) / wall_s if wall_s > 0 else float("nan")
    return out


def generate_prompt(tokenizer, n_tokens: int, seed: int = 0) -> str:
    """A prompt that encodes to exactly n_tokens tokens (adjusts and re-encodes until it does)."""
    rng = random.Random(seed)
    vocab = tokenizer.vocab_size
    ids = [rng.randrange(1000, max(vocab - 1000, 1001)) for _ in range(n_tokens)]
    for _ in range(8):
        text = tokenizer.decode(ids)
        got = tokenizer.encode(text, add_special_tokens=False)
        if len(got) == n_tokens:
            return text
        ids = (got + [rng.randrange(1000, max(vocab - 1000, 1001)) for _ in range(n_tokens)])[:n_tokens]
    # no fixed point within the rounds (a tokenizer whose merges keep shifting): never return more than asked for
    while ids and len(tokenizer.encode(tokenizer.decode(ids), add_special_tokens=False)) > n_tokens:
        ids = ids[:-1]
    return tokenizer.decode(ids)


def _lognormal(rng: random.Random, median: float, sigma: float, lo: int, hi: int) -> int:
    return int(min(max(rng.lognormvariate(math.log(median), sigma), lo), hi))


def synthetic_chat_trace(n: int, rate: float, seed: int = 0, prompt_median: int = 600, output_median: int = 300,
                         shared_fraction: float = 0.3, shared_prefix_tokens: int = 512,
                         word: str = "hello ") -> List[TraceItem]:
    """Poisson arrivals at `rate` req/s; prompt lengths lognormal(median 600) clipped to [16, 16384]; output lengths
    lognormal(median 300) clipped to [1, 4096]; `shared_fraction` of requests start with the same prefix."""
    rng = random.Random(seed)
    t, items = 0.0, []
    prefix = "".join(f"ctx{rng.randrange(10**6)} " for _ in range(shared_prefix_tokens // 2))
    for i in range(n):
        t += rng.expovariate(rate)
        n_in = _lognormal(rng, prompt_median, 1.0, 16, 16384)
        n_out = _lognormal(rng, output_median, 1.0, 1, 4096)
        body = "".join(f"w{rng.randrange(10**6)} " for _ in range(max(n_in // 2, 1)))
        prompt = (prefix + body) if rng.random() < shared_fraction else body
        items.append(TraceItem(t, prompt, n_out, n_in))
    return items


def read_qwen_trace(path: str, limit: Optional[int] = None) -> List[TraceItem]:
    """jsonl with chat_id / timestamp / input_length / output_length (Qwen bailian trace)."""
    items = []
    with open(path) as f:
        for line in f:
            j = json.loads(line)
            n_in, n_out = int(j.get("input_length", 0)), int(j.get("output_length", 1))
            items.append(TraceItem(float(j.get("timestamp", 0.0)), "x " * max(n_in, 1), max(n_out, 1), n_in))
            if limit and len(items) >= limit:
                break
    t0 = min(i.arrival_s for i in items) if items else 0.0
    for i in items:
        i.arrival_s -= t0
    return items


def read_mooncake_trace(path: str, limit: Optional[int] = None) -> List[TraceItem]:
    """jsonl with timestamp (ms) / input_length / output_length (Mooncake trace)."""
    items = read_qwen_trace(path, limit)
    for i in items:
        i.arrival_s /= 1000.0
    return items


def scale_traces(items: Sequence[TraceItem], factor: float) -> List[TraceItem]:
    """factor > 1 compresses time (higher request rate)."""
    return [TraceItem(i.arrival_s / factor, i.prompt, i.output_len, i.input_len) for i in items]


async def _one(client, url: str, model: str, item: TraceItem, t_zero: float, extra: dict) -> RequestResult:
    await asyncio.sleep(max(t_zero + item.arrival_s - time.perf_counter(), 0))
    res = RequestResult(t_start=time.perf_counter())
    body = {"model": model, "messages": [{"role": "user", "content": item.prompt}], "max_tokens": item.output_len,
            "stream": True, "ignore_eos": True, **extra}
    try:
        async with client.stream("POST", url + "/v1/chat/completions", json=body, timeout=None) as r:
            if r.status_code != 200:
                res.ok = False
                return res
            async for line in r.aiter_lines():
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ch = json.loads(line[6:])
                if ch.get("choices") and (ch["choices"][0]["delta"].get("content") or
                                          ch["choices"][0]["delta"].get("reasoning_content")):
                    res.tics.append(time.perf_counter())
    except Exception:
        res.ok = False
    return res


async def benchmark_trace(url: str, model: str, items: Sequence[TraceItem], extra: Optional[dict] = None) -> Dict[str, Any]:
    import httpx

    async with httpx.AsyncClient(limits=httpx.Limits(max_connections=None)) as client:
        t0 = time.perf_counter()
        results = await asyncio.gather(*[_one(client, url, model, it, t0, extra or {}) for it in items])
        return summarize(results, time.perf_counter() - t0)
