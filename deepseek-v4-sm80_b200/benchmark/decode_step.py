"""Device time of one decode forward on one GPU, with the per-rank shapes of an N-way tensor/expert-parallel run.

    python -m minisgl.benchmark.decode_step --layers 4 --tp 8 --batch 128 --context 1024 [--graph 1]

The model is built with the weight shards of rank 0 of ``--tp`` ranks (random weights); collectives are skipped, so
the number is the compute part of a rank's step.  With ``--graph 1`` the step is captured in a CUDA graph and replayed
(launch overhead amortised, as the engine does); the kernel list of the eager steps is what
``ncu --metrics gpu__time_duration.sum`` captures.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json

import torch


class _Slots:
    """One request per table slot, pages handed out sequentially."""

    def __init__(self, model, pool, cfg, device, page_size, num_slots, max_len):
        self.model, self.pool, self.cfg, self.device, self.ps = model, pool, cfg, device, page_size
        self.page_table = torch.zeros(num_slots + 1, max_len, dtype=torch.int32, device=device)
        self.pages, self.lens = {}, {}

    def _ensure(self, slot, upto):
        have = self.pages.setdefault(slot, [])
        need = (upto + self.ps - 1) // self.ps
        if need > len(have):
            new = self.pool.alloc_pages(need - len(have))
            start = len(have) * self.ps
            have.extend(new)
            locs = torch.cat([torch.arange(p * self.ps, (p + 1) * self.ps) for p in new]).to(torch.int32)
            self.page_table[slot, start:start + len(locs)] = locs.to(self.device)

    def batch(self, chunks):
        from minisgl.models.deepseek_v4 import ForwardBatch

        ids, pos, slots, last = [], [], [], []
        for slot, toks in chunks:
            n0 = self.lens.get(slot, 0)
            self._ensure(slot, n0 + len(toks))
            ids += list(toks)
            pos += list(range(n0, n0 + len(toks)))
            slots += [slot] * len(toks)
            last.append(len(ids) - 1)
            self.lens[slot] = n0 + len(toks)
        dev = self.device
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        slot_t = torch.tensor(slots, dtype=torch.int32, device=dev)
        out_loc = self.page_table[slot_t.long(), pos_t.long()]
        return ForwardBatch(torch.tensor(ids, dtype=torch.int32, device=dev), pos_t, slot_t, out_loc,
                            torch.tensor(last, dtype=torch.int64, device=dev), self.page_table,
                            is_prefill=any(len(t) > 1 for _, t in chunks), max_context=max(self.lens.values()))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--graph", type=int, default=1)
    ap.add_argument("--profile", type=int, default=0, help="print the per-launcher share of the eager steps")
    a = ap.parse_args(argv)
    from minisgl.kvcache.pool import DSV4KVPool, PoolSizes
    from minisgl.models import synth
    from minisgl.models.config import ModelConfig
    from minisgl.models.deepseek_v4 import Comm, DSV4Model
    from minisgl.ops import native

    dev = torch.device("cuda")
    cfg = ModelConfig.flash().with_layers(a.layers)
    w = synth.random_weights(cfg, dev, rank=0, size=a.tp, moe_mode="ep", fast_experts=True)

    class ShardOnly(Comm):  # shard shapes of rank 0 of `tp`, no collectives
        rank, size = 0, a.tp

    ps = 256
    pages = a.batch * ((a.context + 64) // ps + 2)
    pool = DSV4KVPool(cfg, PoolSizes(pages, pages, a.batch, ps), dev)
    model = DSV4Model(cfg, w, pool, ShardOnly() if a.tp > 1 else None, "ep")
    slots = _Slots(model, pool, cfg, dev, ps, a.batch, ((a.context + 128) // ps + 2) * ps)
    g = torch.Generator().manual_seed(0)
    per = max(1, 8192 // a.context)
    starts = list(range(0, a.batch, per))
    prefill_ms, prefill_share = [], None
    for s0 in starts:
        fb = slots.batch([(s, torch.randint(0, cfg.vocab_size, (a.context,), generator=g).tolist())
                          for s in range(s0, min(s0 + per, a.batch))])
        torch.cuda.synchronize()
        last = a.profile and s0 == starts[-1]
        if last:  # per-launcher share of the last prefill forward (all its chunks' caches are warm by then)
            native.enable_profile(True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.forward(fb)
        e1.record()
        torch.cuda.synchronize()
        prefill_ms.append(e0.elapsed_time(e1))
        if last:
            rep = native.profile_report()
            native.enable_profile(False)
            prefill_share = {k: round(t, 3) for k, (c, t) in list(rep.items())[:14]}
    torch.cuda.synchronize()
    n0 = native.launch_count()
    if a.profile:
        native.enable_profile(True)
    for _ in range(a.steps):
        fb = slots.batch([(s, [5]) for s in range(a.batch)])
        model.forward(fb)
    torch.cuda.synchronize()
    launches = (native.launch_count() - n0) / a.steps
    out = {"layers": a.layers, "tp": a.tp, "batch": a.batch, "context": a.context, "launches_per_step": launches,
           "prefill_tokens_per_forward": min(per, a.batch) * a.context,
           "prefill_ms_per_forward": round(sorted(prefill_ms)[len(prefill_ms) // 2], 3)}
    if prefill_share is not None:
        out["prefill_share_ms"] = prefill_share
    if a.profile:
        rep = native.profile_report()
        native.enable_profile(False)
        out["eager_share_ms"] = {k: round(t / a.steps, 3) for k, (c, t) in list(rep.items())[:12]}
    if a.graph:
        fb = slots.batch([(s, [5]) for s in range(a.batch)])
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            model.forward(fb)
        st.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            model.forward(fb)
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        out["graph_ms_per_step"] = round(ms, 4)
        out["graph_us_per_layer"] = round(ms * 1e3 / a.layers, 1)
    native.assert_device_ok()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
