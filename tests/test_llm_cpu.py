"""End to end on CPU: the offline LLM (scheduler + engine + model on the PyTorch oracle) with the tiny model --
4 prompts of 64 random tokens, page size 16, greedy decode of 16 tokens -- must reproduce, token for token, a plain
loop that feeds the model one request at a time without the scheduler."""
import torch

from helpers import MiniRunner
from minisgl.core import SamplingParams
from minisgl.llm import LLM
from minisgl.models.config import ModelConfig


def _prompts(n=4, length=64, vocab=1024):
    g = torch.Generator().manual_seed(0)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _reference_tokens(cfg, prompt, n_out, ps):
    r = MiniRunner(cfg, page_size=ps, num_pages=32, seed=0)
    out = []
    logits = r.step([(0, prompt)])
    for _ in range(n_out):
        t = int(logits.argmax(-1)[0])
        out.append(t)
        logits = r.step([(0, [t])])
    return out


def test_offline_generate_matches_plain_loop():
    cfg = ModelConfig.tiny()
    llm = LLM(model_config=cfg, device="cpu", page_size=16, max_running_req=4, num_page_override=64, seed=0,
              use_dummy_weight=True, disable_log_stats=True)
    prompts = _prompts()
    outs = llm.generate(prompts, SamplingParams(max_tokens=16, ignore_eos=True))
    assert [len(o.token_ids) for o in outs] == [16] * 4
    assert all(o.finish_reason == "length" for o in outs)
    for p, o in zip(prompts[:2], outs[:2]):
        assert o.token_ids == _reference_tokens(cfg, p, 16, 16)
    llm.engine.pool.assert_no_leak() if llm.cache.radix is None else None
    # every request slot and window pin is back
    assert llm.table.available_size == 4
    assert not llm.pending_retire and not llm.decode.running


def test_prefix_reuse_gives_same_tokens():
    cfg = ModelConfig.tiny()
    llm = LLM(model_config=cfg, device="cpu", page_size=16, max_running_req=2, num_page_override=64, seed=0,
              use_dummy_weight=True, disable_log_stats=True)
    g = torch.Generator().manual_seed(5)
    shared = torch.randint(0, 1024, (160,), generator=g).tolist()
    a = shared + [7, 8, 9]
    b = shared + [11, 12]
    first = llm.generate([a], SamplingParams(max_tokens=4, ignore_eos=True))[0]
    hit0 = llm.cache.radix.metrics["hit_tokens"]
    second = llm.generate([b], SamplingParams(max_tokens=4, ignore_eos=True))[0]
    assert llm.cache.radix.metrics["hit_tokens"] - hit0 == 128  # 160 shared tokens -> the 128-aligned boundary
    assert second.token_ids == _reference_tokens(cfg, b, 4, 16)
    assert first.token_ids == _reference_tokens(cfg, a, 4, 16)
    # structured reports: weight preparation and window-storage residency
    rep = llm.engine.model_prepare_report
    assert rep["bytes_total"] == sum(rep["bytes_by_format"].values()) > 0 and rep["experts_local"] == 8
    assert {"fp4_packed", "e8m0_scales", "float8_e4m3fn"} <= set(rep["bytes_by_format"])
    swa = llm.engine.pool.runtime_swa_counters()
    assert swa["swa_slots_in_use"] + swa["swa_slots_free"] == swa["swa_slots_total"]
    assert swa["swa_taken"] - swa["swa_released"] == swa["swa_slots_in_use"]
    assert swa["pages_pinned_by_tree"] > 0  # the cached prefix keeps its window rows
