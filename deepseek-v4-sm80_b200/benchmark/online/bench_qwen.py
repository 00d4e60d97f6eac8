"""Trace replay against a running server at several time scales (benchmark/online/bench_qwen.py of the reference
replays the Qwen trace at 6 scales).  ``--trace`` is a Qwen- or Mooncake-format jsonl; without it the synthetic
chat trace is used: 2 000 requests, Poisson arrivals at each of the given rates, log-normal prompt (median 600) and
output (median 300) lengths, 30 % of the requests sharing a 512-token prefix."""
from __future__ import annotations

import argparse
import asyncio
import json

from minisgl.benchmark.client import (benchmark_trace, read_mooncake_trace, read_qwen_trace, scale_traces,
                                      synthetic_chat_trace)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:1919")
    ap.add_argument("--model", required=True)
    ap.add_argument("--trace", default="")
    ap.add_argument("--format", default="qwen", choices=["qwen", "mooncake"])
    ap.add_argument("--scales", type=float, nargs="+", default=[0.5, 1, 2, 4, 8, 16])
    ap.add_argument("--rates", type=float, nargs="+", default=[1, 4, 16, 64])
    ap.add_argument("-n", type=int, default=2000)
    a = ap.parse_args(argv)
    runs = []
    if a.trace:
        base = (read_qwen_trace if a.format == "qwen" else read_mooncake_trace)(a.trace, a.n)
        runs = [(f"scale {s}", scale_traces(base, s)) for s in a.scales]
    else:
        runs = [(f"rate {r} req/s", synthetic_chat_trace(a.n, r)) for r in a.rates]
    for name, items in runs:
        res = asyncio.run(benchmark_trace(a.url, a.model, items))
        print(name, json.dumps({k: res[k] for k in ("ttft", "tpot", "output_tok_s", "req_s", "failed")}))


if __name__ == "__main__":
    main()
