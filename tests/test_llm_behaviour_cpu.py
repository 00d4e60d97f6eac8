"""Scheduler behaviour end to end on CPU (tiny model, PyTorch oracle): staggered arrivals give the same tokens as a
single wave, EOS ends a request with ``stop``, an abort in mid-generation returns every resource and leaves the
other requests untouched, over-long prompts are rejected and over-long output budgets clipped."""
import torch

from minisgl.core import SamplingParams
from minisgl.llm import LLM
from minisgl.message import AbortBackendMsg
from minisgl.models.config import ModelConfig


def _llm(**kw):
    base = dict(model_config=ModelConfig.tiny(), device="cpu", page_size=16, max_running_req=4, num_page_override=64,
                seed=0, use_dummy_weight=True, disable_log_stats=True)
    base.update(kw)
    return LLM(**base)


def _prompts(n, length, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _idle(llm):
    assert llm.table.available_size == llm.config.max_running_req
    assert not llm.decode.running and not llm.prefill.runnable and not llm.pending_retire


def test_staggered_arrivals_match_the_single_wave():
    prompts = _prompts(4, 48, seed=1)
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    wave = _llm().generate(prompts, sp)
    llm = _llm()
    late = llm.generate(prompts, sp, arrival_gap_steps=3)
    assert [o.token_ids for o in late] == [o.token_ids for o in wave]
    steps = llm.phase_steps
    assert steps["prefill"] >= 3 and steps["decode"] > 12      # arrivals were spread over the decode of earlier ones
    _idle(llm)


def test_eos_stops_a_request_and_ignore_eos_does_not():
    prompts = _prompts(2, 40, seed=2)
    free = _llm().generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    # make the 4th token of the first request the end-of-sequence id
    eos = free[0].token_ids[3]
    cut = free[0].token_ids.index(eos) + 1                      # it may occur earlier by chance
    llm = _llm()
    llm.eos_token_id = eos
    outs = llm.generate(prompts, [SamplingParams(max_tokens=10), SamplingParams(max_tokens=10, ignore_eos=True)])
    assert outs[0].finish_reason == "stop" and outs[0].token_ids == free[0].token_ids[:cut]
    assert outs[1].finish_reason == "length" and outs[1].token_ids == free[1].token_ids
    _idle(llm)


def test_abort_in_mid_generation_returns_resources_and_spares_the_others():
    prompts = _prompts(3, 40, seed=3)
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    want = _llm().generate(prompts, sp)
    llm = _llm()
    polls = {"n": 0}
    real = llm.receive_msg

    def receive(blocking):
        polls["n"] += 1
        msgs = real(blocking)
        if polls["n"] == 6:                                     # the wave is decoding by now
            msgs = list(msgs) + [AbortBackendMsg(1)]
        return msgs

    llm.receive_msg = receive
    outs = llm.generate(prompts, sp)
    assert outs[1].finish_reason == "abort" and 0 < len(outs[1].token_ids) < 16
    assert outs[1].token_ids == want[1].token_ids[:len(outs[1].token_ids)]
    assert outs[0].token_ids == want[0].token_ids and outs[2].token_ids == want[2].token_ids
    assert outs[0].finish_reason == outs[2].finish_reason == "length"
    _idle(llm)
    if llm.cache.radix is not None:
        llm.cache.radix.reset()
    llm.engine.pool.assert_no_leak()


def test_over_long_prompt_is_rejected_and_output_budget_is_clipped():
    llm = _llm(context_length=128)
    limit = llm.engine.max_seq_len
    ok = _prompts(1, limit - 5, seed=4)[0]
    too_long = _prompts(1, limit, seed=5)[0]
    outs = llm.generate([too_long, ok], SamplingParams(max_tokens=50, ignore_eos=True))
    assert outs[0].finish_reason == "length_rejected" and outs[0].token_ids == []
    assert outs[1].finish_reason == "length" and len(outs[1].token_ids) == 5   # clipped to the sequence limit
    _idle(llm)
