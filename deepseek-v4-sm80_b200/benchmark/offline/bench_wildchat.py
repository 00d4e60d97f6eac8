"""Offline benchmark over chat-style prompts of mixed lengths with temperature sampling
(benchmark/offline/bench_wildchat.py of the reference: 256 WildChat prompts, temperature 0.6).  Without network
access the prompts come from a jsonl file (``--data``, one {"prompt": ...} or {"conversation": [...]} per line) or,
by default, from a synthetic length distribution with the same median."""
from __future__ import annotations

import argparse
import json
import random
import time


def load_prompts(path, n, vocab, seed=0, max_len=4096):
    import torch

    rng = random.Random(seed)
    if path:
        rows = [json.loads(l) for l in open(path)][:n]
        return [r.get("prompt") or r["conversation"] for r in rows]
    g = torch.Generator().manual_seed(seed)
    lens = [int(min(max(rng.lognormvariate(5.5, 1.0), 8), max_len)) for _ in range(n)]
    return [torch.randint(0, vocab, (l,), generator=g, dtype=torch.int32) for l in lens]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--data", default="")
    ap.add_argument("-n", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tiny", action="store_true", help="tiny architecture (CPU-sized) with random weights")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--page-size", type=int, default=256)
    ap.add_argument("--num-pages", type=int, default=0, help="override the KV page count (CPU runs need it)")
    ap.add_argument("--max-prompt", type=int, default=4096, help="clip of the synthetic prompt lengths")
    a = ap.parse_args(argv)
    from minisgl.core import SamplingParams
    from minisgl.llm import LLM
    from minisgl.models.config import ModelConfig

    kw = {}
    if a.tiny:
        kw = dict(model_config=ModelConfig.tiny(), use_dummy_weight=True)
    elif not a.model:
        kw = dict(model_config=ModelConfig.flash().with_layers(a.layers), use_dummy_weight=True)
    if a.num_pages:
        kw["num_page_override"] = a.num_pages
    llm = LLM(a.model, recipe="default_m128", device=a.device, page_size=a.page_size, **kw)
    prompts = load_prompts(a.data, a.n, llm.engine.model_config.vocab_size, max_len=a.max_prompt)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, SamplingParams(temperature=a.temperature, max_tokens=a.max_tokens))
    dt = time.perf_counter() - t0
    res = {"requests": len(outs), "wall_s": dt, "output_tok_s": sum(len(o.token_ids) for o in outs) / dt,
           "finish_reasons": sorted({o.finish_reason for o in outs})}
    if llm.tp.is_primary():
        print(res)
    llm.shutdown()
    return res


if __name__ == "__main__":
    main()
