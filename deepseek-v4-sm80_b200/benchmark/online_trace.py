"""Online-serving trace through the engine: Poisson arrivals in wall-clock time against a running scheduler.

    python -m minisgl.benchmark.online_trace --dummy --layers 4 --requests 256 --rates 4 16 64 --recipe high_m256

The workload is the synthetic chat trace of ``minisgl.benchmark.client.synthetic_chat_trace`` in token form: arrival
times from a Poisson process at ``rate`` requests per second, prompt lengths log-normal (median 600, clipped to
[16, 16384]), output lengths log-normal (median 300, clipped to [1, 4096]), and 30 % of the prompts starting with
one common 512-token prefix so that the radix cache is exercised.  Requests become visible to the scheduler when
their arrival time has passed -- the offline ``LLM`` with a clock-driven message source instead of a list -- so
admission, mixed prefill / decode phases, prefix hits and overlap scheduling behave as they do behind the HTTP
server; the tokenizer and HTTP layers are left out (they need a tokenizer file, which a random-init run lacks; the
same trace against a served model is ``minisgl.benchmark.online.bench_simple``).  Reports p50 / p90 / p99 TTFT and
TPOT, output tok/s and req/s per rate.  Counterpart of the reference's online benchmarks
(python/minisgl/benchmark/client.py:18-498, benchmark/online/*.py).
"""
from __future__ import annotations

import argparse
import json
import math
import random
import time
from typing import List

import torch


def token_trace(n: int, rate: float, vocab: int, seed: int = 0, prompt_median: int = 600, output_median: int = 300,
                shared_fraction: float = 0.3, shared_prefix_tokens: int = 512, max_prompt: int = 16384,
                max_output: int = 4096):
    """[(arrival seconds, prompt token ids int32 tensor, output length)]"""
    rng = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    prefix = torch.randint(0, vocab, (shared_prefix_tokens,), generator=g, dtype=torch.int32)
    t, out = 0.0, []
    for _ in range(n):
        t += rng.expovariate(rate)
        n_in = int(min(max(rng.lognormvariate(math.log(prompt_median), 1.0), 16), max_prompt))
        n_out = int(min(max(rng.lognormvariate(math.log(output_median), 1.0), 1), max_output))
        body = torch.randint(0, vocab, (n_in,), generator=g, dtype=torch.int32)
        if rng.random() < shared_fraction:
            body = torch.cat([prefix, body])[:max_prompt]
        out.append((t, body, n_out))
    return out


def make_timed_llm(base_cls):
    class TimedLLM(base_cls):
        """``LLM`` whose requests appear when their arrival time has passed."""

        def start_trace(self, trace, sampling):
            from minisgl.message import UserMsg

            self._trace = sorted(trace, key=lambda x: x[0])
            self._next = 0
            self._t_zero = time.perf_counter()
            self._arrival = {}
            self._uid0 = self._next_uid
            self._timed = True
            self._open = len(trace)
            for i, (ta, ids, n_out) in enumerate(self._trace):
                uid = self._next_uid
                self._next_uid += 1
                from minisgl.core import SamplingParams
                from minisgl.llm.llm import RequestOutput

                self._results[uid] = RequestOutput(uid)
                self._arrival[uid] = ta
                self._trace[i] = (ta, UserMsg(uid, ids, SamplingParams(max_tokens=n_out, **sampling), None))

        def receive_msg(self, blocking: bool):
            from minisgl.scheduler.scheduler import RequestAllFinished

            if not getattr(self, "_timed", False):
                return super().receive_msg(blocking)
            if self._next >= len(self._trace):
                if self._open == 0:
                    raise RequestAllFinished()
                return []
            now = time.perf_counter() - self._t_zero
            out = []
            while self._next < len(self._trace) and self._trace[self._next][0] <= now:
                out.append(self._trace[self._next][1])
                self._next += 1
            if not out and blocking:
                # idle until the next arrival
                time.sleep(max(min(self._trace[self._next][0] - now, 0.05), 0.0))
            return out

        def run_trace(self, trace, sampling=None) -> dict:
            from minisgl.scheduler.scheduler import RequestAllFinished

            self.start_trace(trace, sampling or {"ignore_eos": True})
            try:
                last = None
                while True:
                    last = self.overlap_loop(last)
            except RequestAllFinished:
                pass
            self._timed = False
            wall = time.perf_counter() - self._t_zero
            uids = list(self._arrival)
            outs = [self._results.pop(u) for u in uids]
            ttft, tpot, n_tok = [], [], 0
            for u, o in zip(uids, outs):
                n_tok += len(o.token_ids)
                if o.t_first is not None:
                    ttft.append(o.t_first - (self._t_zero + self._arrival[u]))
                if len(o.t_tokens) > 1:
                    tpot.append((o.t_tokens[-1] - o.t_tokens[0]) / (len(o.t_tokens) - 1))
            from minisgl.benchmark.client import percentile

            def stats(xs, scale=1.0):
                return {k: round(percentile(xs, p) * scale, 4) for k, p in (("p50", 50), ("p90", 90), ("p99", 99))}

            return {"requests": len(outs), "finished": sum(o.finish_reason == "length" for o in outs),
                    "wall_s": round(wall, 3), "output_tokens": n_tok, "output_tok_s": round(n_tok / wall, 1),
                    "req_s": round(len(outs) / wall, 3), "ttft_s": stats(ttft), "tpot_ms": stats(tpot, 1e3),
                    "prefix": {k: v for k, v in self.cache.prefix_metrics_snapshot().items()
                               if k in ("hit_tokens", "query_tokens", "hit_rate", "evicted_pages", "dedup_pages")}}

    return TimedLLM


def main(argv=None) -> List[dict]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--recipe", default="high_m256")
    ap.add_argument("--requests", type=int, default=2000)
    ap.add_argument("--rates", type=float, nargs="+", default=[1, 4, 16, 64])
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--page-size", type=int, default=256)
    ap.add_argument("--num-pages", type=int, default=0)
    ap.add_argument("--max-running", type=int, default=0)
    ap.add_argument("--prompt-median", type=int, default=600)
    ap.add_argument("--output-median", type=int, default=300)
    ap.add_argument("--max-prompt", type=int, default=16384)
    ap.add_argument("--max-output", type=int, default=4096)
    ap.add_argument("--graph-bs", type=int, nargs="*", default=None)
    a = ap.parse_args(argv)
    import dataclasses

    from minisgl.llm import LLM
    from minisgl.models.config import ModelConfig

    kw = {}
    if a.tiny or a.dummy or not a.model:
        cfg = ModelConfig.tiny() if a.tiny else ModelConfig.flash()
        cfg = cfg.with_layers(a.layers) if a.layers else cfg
        if a.experts:
            cfg = dataclasses.replace(cfg, n_routed_experts=a.experts)
        kw = dict(model_config=cfg, use_dummy_weight=True)
    if a.num_pages:
        kw["num_page_override"] = a.num_pages
    if a.max_running:
        kw["max_running_req"] = a.max_running
    if a.graph_bs is not None:
        kw["cuda_graph_bs"] = a.graph_bs
    llm = make_timed_llm(LLM)(a.model, recipe=a.recipe if not a.max_running else None, device=a.device,
                              page_size=a.page_size, context_length=a.max_prompt + a.max_output + 64,
                              disable_log_stats=True, **kw)
    vocab = llm.engine.model_config.vocab_size
    results = []
    for rate in a.rates:
        trace = token_trace(a.requests, rate, vocab, seed=int(rate * 1000) + 1, prompt_median=a.prompt_median,
                            output_median=a.output_median, max_prompt=a.max_prompt, max_output=a.max_output)
        res = {"rate_req_s": rate, **llm.run_trace(trace)}
        results.append(res)
        if llm.tp.is_primary():
            print(json.dumps(res), flush=True)
        if llm.cache.radix is not None:
            llm.cache.radix.reset()
    llm.shutdown()
    return results


if __name__ == "__main__":
    main()
