"""Online benchmark against a running server: a fixed batch of concurrent chat requests
(benchmark/online/bench_simple.py of the reference: batch 64)."""
from __future__ import annotations

import argparse
import asyncio
import json

from minisgl.benchmark.client import TraceItem, benchmark_trace


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:1919")
    ap.add_argument("--model", required=True)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--input-words", type=int, default=512)
    ap.add_argument("--output-len", type=int, default=256)
    a = ap.parse_args(argv)
    items = [TraceItem(0.0, f"req{i} " + "word " * a.input_words, a.output_len) for i in range(a.batch)]
    print(json.dumps(asyncio.run(benchmark_trace(a.url, a.model, items)), indent=1))


if __name__ == "__main__":
    main()
