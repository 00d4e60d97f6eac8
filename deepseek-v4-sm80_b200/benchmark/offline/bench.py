"""Offline wave benchmark: M sequences, fixed input / output lengths, greedy, ignore-EOS, through ``LLM.generate``
(benchmark/offline/bench.py of the reference: M=128, 1 024 in, 1 024 out).  Run under
``minisgl.distributed.launch_tensor_parallel`` or torchrun for tp > 1.  With ``--dummy`` the model is random-init."""
from __future__ import annotations

import argparse
import time


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("-M", "--batch", type=int, default=128)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=1024)
    ap.add_argument("--recipe", default="default_m128")
    ap.add_argument("--tiny", action="store_true", help="tiny architecture (CPU-sized); implies --dummy")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--page-size", type=int, default=256)
    ap.add_argument("--num-pages", type=int, default=0, help="override the KV page count (CPU runs need it)")
    a = ap.parse_args(argv)
    import torch

    from minisgl.core import SamplingParams
    from minisgl.llm import LLM
    from minisgl.models.config import ModelConfig

    kw = {}
    if a.tiny or a.dummy or not a.model:
        cfg = ModelConfig.tiny() if a.tiny else ModelConfig.flash()
        kw = dict(model_config=cfg.with_layers(a.layers) if a.layers else cfg, use_dummy_weight=True)
    if a.num_pages:
        kw["num_page_override"] = a.num_pages
    llm = LLM(a.model, recipe=a.recipe, max_running_req=a.batch, device=a.device, page_size=a.page_size, **kw)
    vocab = llm.engine.model_config.vocab_size
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, vocab, (a.input_len,), generator=g, dtype=torch.int32) for _ in range(a.batch)]
    t0 = time.perf_counter()
    outs = llm.generate(prompts, SamplingParams(max_tokens=a.output_len, ignore_eos=True))
    dt = time.perf_counter() - t0
    n_out = sum(len(o.token_ids) for o in outs)
    res = {"requests": len(outs), "wall_s": dt, "req_s": len(outs) / dt, "output_tok_s": n_out / dt,
           "prefix": llm.cache.prefix_metrics_snapshot()}
    if llm.tp.is_primary():
        print(res)
    llm.shutdown()
    return res


if __name__ == "__main__":
    main()
