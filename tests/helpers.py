"""Small harness that drives the model directly (no scheduler): one request per table slot, sequential pages."""
import torch

from minisgl.kvcache.pool import DSV4KVPool, PoolSizes
from minisgl.models import synth
from minisgl.models.config import ModelConfig
from minisgl.models.deepseek_v4 import DSV4Model, ForwardBatch


class MiniRunner:
    def __init__(self, cfg: ModelConfig, device="cpu", page_size=16, num_pages=64, num_slots=4, max_len=512,
                 weights=None, comm=None, moe_mode="tp", rank=0, size=1, seed=0):
        self.cfg, self.device, self.ps = cfg, torch.device(device), page_size
        self.pool = DSV4KVPool(cfg, PoolSizes(num_pages, num_pages, num_slots, page_size), device)
        self.weights = weights if weights is not None else synth.random_weights(cfg, device, rank, size, moe_mode, seed)
        self.model = DSV4Model(cfg, self.weights, self.pool, comm, moe_mode)
        self.page_table = torch.zeros(num_slots + 1, max_len, dtype=torch.int32, device=device)
        self.pages = {}
        self.lens = {}

    def _ensure(self, slot, upto):
        have = self.pages.setdefault(slot, [])
        need = (upto + self.ps - 1) // self.ps
        if need > len(have):
            new = self.pool.alloc_pages(need - len(have))
            start = len(have) * self.ps
            have.extend(new)
            locs = torch.cat([torch.arange(p * self.ps, (p + 1) * self.ps) for p in new]).to(torch.int32)
            self.page_table[slot, start:start + len(locs)] = locs.to(self.device)

    def step(self, chunks):
        """chunks: list of (slot, token_ids list) appended at the slot's current length. Returns logits [B,V]."""
        return self.model.forward(self.make_fb(chunks))

    def make_fb(self, chunks):
        """The ForwardBatch of ``step`` (pages allocated, lengths advanced) without running the model."""
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
