"""Pure scheduling contracts: fair prefill chunking, the mixed-phase policy, sequence admission, request lifecycle,
graph bucket policy and memory planner, KV pool / radix tree ownership, detokenizer, reasoning states."""
import numpy as np
import pytest
import torch

from minisgl.core import FlightLedger, Req, SamplingParams
from minisgl.engine import graph_memory
from minisgl.engine.graph_policy import default_buckets, pick_bucket, resolve_graph_buckets
from minisgl.kvcache.pool import DSV4KVPool, PoolSizes, bytes_per_page
from minisgl.kvcache.radix_cache import RadixPrefixCache, first_mismatch
from minisgl.models.config import ModelConfig
from minisgl.reasoning import (ReasoningState, advance_reasoning_state, effective_reasoning_state,
                               initial_reasoning_state)
from minisgl.scheduler.phase_policy import MixedPhaseFairPolicy
from minisgl.scheduler.prefill import allocate_fair_prefill_chunks as fair
from minisgl.scheduler.scheduler import decide_max_sequence_admission
from minisgl.scheduler.stats import StatsTracker
from minisgl.tokenizer.detokenize import DetokenizeManager, printable_prefix


# ---------------------------------------------------------------------------- fair chunks
def test_fair_chunks_first_share_then_least_progress():
    assert fair(token_budget=8192, alignment_quantum=256, scheduled_tokens=[0], remaining_tokens=[100000]) == [8192]
    g = fair(token_budget=1024, alignment_quantum=256, scheduled_tokens=[0, 0, 0], remaining_tokens=[5000, 5000, 5000])
    assert g == [512, 256, 256]  # every request first, the remaining quantum to the FIFO head
    g = fair(token_budget=768, alignment_quantum=256, scheduled_tokens=[4096, 0], remaining_tokens=[5000, 5000])
    assert g == [256, 512]  # the spare quantum goes to the request with less granted progress
    g = fair(token_budget=2048, alignment_quantum=256, scheduled_tokens=[0, 0], remaining_tokens=[300, 10000])
    assert g == [300, 1536] and sum(g) <= 2048  # a final tail may be a sub-quantum grant
    g = fair(token_budget=512, alignment_quantum=256, scheduled_tokens=[0, 0, 0], remaining_tokens=[900, 900, 900])
    assert g == [256, 256, 0]
    assert fair(token_budget=100, alignment_quantum=256, scheduled_tokens=[0], remaining_tokens=[900]) == [100]
    with pytest.raises(ValueError):
        fair(token_budget=0, alignment_quantum=256, scheduled_tokens=[0], remaining_tokens=[1])


def test_fair_chunks_never_exceed_budget_random():
    rng = np.random.default_rng(0)
    for _ in range(200):
        n = int(rng.integers(1, 9))
        rem = [int(x) for x in rng.integers(1, 20000, n)]
        sch = [int(x) for x in rng.integers(0, 5000, n)]
        budget = int(rng.choice([256, 2048, 8192]))
        g = fair(token_budget=budget, alignment_quantum=256, scheduled_tokens=sch, remaining_tokens=rem)
        assert sum(g) <= budget and all(0 <= a <= b for a, b in zip(g, rem))
        assert g[0] > 0


# ---------------------------------------------------------------------------- phase policy
def test_mixed_phase_policy_sequence():
    p = MixedPhaseFairPolicy(isolated_prefill_budget=8192)
    assert p.choose(prefill_runnable=True, decode_runnable=False).prefill_budget == 8192
    assert p.choose(prefill_runnable=False, decode_runnable=True).phase == "decode"
    assert p.choose(prefill_runnable=False, decode_runnable=False).phase is None
    seq = []
    for _ in range(12):
        d = p.choose(prefill_runnable=True, decode_runnable=True)
        seq.append(d.phase)
        if d.phase == "prefill":
            assert d.prefill_budget == 2048 and d.mixed
        p.record_scheduled(d.phase, prefill_runnable=True, decode_runnable=True)
    assert seq == ["decode"] * 4 + ["prefill"] + ["decode"] * 4 + ["prefill"] + ["decode"] * 2
    p.record_scheduled("decode", prefill_runnable=False, decode_runnable=True)  # conflict over: state resets
    assert p.snapshot()["mixed_active"] is False
    # a batch that was not built does not consume a fairness slot
    p.record_scheduled(None, prefill_runnable=True, decode_runnable=True)
    assert p.choose(prefill_runnable=True, decode_runnable=True).phase == "decode"
    with pytest.raises(ValueError):
        MixedPhaseFairPolicy(isolated_prefill_budget=0)


def test_sequence_admission():
    assert decide_max_sequence_admission(100, 50, 1000) == (True, 50, "")
    assert decide_max_sequence_admission(990, 50, 1000)[:2] == (True, 10)
    ok, _, why = decide_max_sequence_admission(1000, 5, 1000)
    assert not ok and "exceeds" in why
    assert not decide_max_sequence_admission(0, 5, 1000)[0]


# ---------------------------------------------------------------------------- lifecycle
def test_lifecycle_defers_release_until_all_forwards_complete():
    lc = FlightLedger(admission=7)
    t0, t1 = lc.launch(), lc.launch()
    lc.end("stop")
    assert not lc.may_release and not lc.is_open and lc.in_flight == 2
    with pytest.raises(RuntimeError):
        lc.launch()
    with pytest.raises(RuntimeError):
        lc.land(7, t1)                      # forwards land in launch order
    lc.land(7, t0)
    assert not lc.may_release
    with pytest.raises(RuntimeError):
        lc.land(8, t1)                      # a landing of another admission
    lc.land(7, t1)
    assert lc.may_release and lc.in_flight == 0
    lc.released()
    assert lc.phase == "closed"
    with pytest.raises(RuntimeError):
        lc.released()
    with pytest.raises(RuntimeError):
        lc.end("again")


def test_req_host_buffer_and_counters():
    r = Req(torch.arange(5, dtype=torch.int32), 0, 0, 3, 1, SamplingParams(max_tokens=3))
    assert (r.extend_len, r.remain_len, r.can_decode) == (5, 3, True)
    r.complete_one()
    assert (r.cached_len, r.device_len) == (5, 6)
    for t in (9, 8, 7):
        r.append_host(torch.tensor([t], dtype=torch.int32))
    assert r.input_ids.tolist() == [0, 1, 2, 3, 4, 9, 8, 7] and not r.can_commit_token
    with pytest.raises(RuntimeError):
        r.append_host(torch.tensor([1], dtype=torch.int32))
    with pytest.raises(ValueError):
        r.append_host(torch.tensor([1], dtype=torch.int64))
    assert SamplingParams(temperature=0.7, top_k=1).is_greedy and not SamplingParams(temperature=0.0, top_p=0.9).is_greedy


# ---------------------------------------------------------------------------- graphs
def test_graph_bucket_policy():
    assert default_buckets(128) == [1, 2, 4] + list(range(8, 129, 8))
    b = default_buckets(300)
    assert b[-1] == 300 and 272 in b and 288 in b and 264 not in b
    p = resolve_graph_buckets(max_running_req=128)
    assert p.mode == "release_default" and p.max_bs == 128
    assert resolve_graph_buckets(max_running_req=1000).max_bs == 512
    assert resolve_graph_buckets(max_running_req=64, explicit_max=16).buckets == (1, 2, 4, 8, 16)
    assert resolve_graph_buckets(max_running_req=64, explicit_list=[8, 2, 8]).buckets == (2, 8)
    assert resolve_graph_buckets(max_running_req=64, explicit_max=0).mode == "disabled"
    assert resolve_graph_buckets(max_running_req=64, enabled=False).buckets == ()
    with pytest.raises(ValueError):
        resolve_graph_buckets(max_running_req=8, explicit_list=[16])
    with pytest.raises(ValueError):
        resolve_graph_buckets(max_running_req=8, explicit_max=9)
    assert pick_bucket((1, 2, 4, 8), 3) == 4 and pick_bucket((1, 2), 3) is None


def test_graph_memory_planner():
    est = graph_memory.estimate_graph_memory(buckets=(1, 2, 4, 8), num_context_classes=3, hidden_size=4096)
    assert est.num_graphs == 12 and est.reserve_bytes == est.estimate_bytes + est.margin_bytes
    assert graph_memory.estimate_graph_memory(buckets=(), num_context_classes=3, hidden_size=4096).reserve_bytes == 0
    assert graph_memory.select_num_pages(budget_bytes=1000, bytes_per_page=10) == 100
    assert graph_memory.select_num_pages(budget_bytes=1000, bytes_per_page=10, override=50) == 50
    with pytest.raises(RuntimeError):
        graph_memory.select_num_pages(budget_bytes=1000, bytes_per_page=10, override=101)
    with pytest.raises(RuntimeError):
        graph_memory.select_num_pages(budget_bytes=5, bytes_per_page=10)
    assert graph_memory.compare_graph_capture(est, est.estimate_bytes)["overrun_bytes"] == 0
    with pytest.raises(RuntimeError):
        graph_memory.compare_graph_capture(est, est.reserve_bytes + 1)


# ---------------------------------------------------------------------------- KV pool + radix
def _pool(pages=16, swa=8, ps=16):
    return DSV4KVPool(ModelConfig.tiny(), PoolSizes(pages, swa, 4, ps), "cpu")


def test_pool_refcounts_swa_lifetime_and_leak_check():
    pool = _pool()
    a = pool.alloc_pages(3)
    assert pool.num_free_pages == 13 and pool.num_free_swa == 5 and all(pool.has_swa(p) for p in a)
    pool.pin_swa(a)
    pool.ref_pages(a[:1])               # the radix tree takes a reference
    pool.unpin_swa(a[:2])               # the window moved past the first two pages
    # nobody pins them: their window rows stay readable until another page needs the slots
    assert all(pool.has_swa(p) for p in a) and pool.num_free_swa == 7
    assert pool.runtime_swa_counters()["swa_slots_reclaimable"] == 2
    b = pool.alloc_pages(6)             # 5 unused slots + the least recently unpinned page's slot
    assert not pool.has_swa(a[0]) and pool.has_swa(a[1]) and pool.counters["swa_reclaimed"] == 1
    assert int(pool.swa_map[a[0]]) == -1 and int(pool.swa_map[a[2]]) >= 0
    with pytest.raises(RuntimeError):
        pool.alloc_pages(2)             # one reclaimable slot left, pages would be there
    pool.pin_swa(a[1:2])                # pinned again: not reclaimable any more
    assert pool.num_free_swa == 0
    pool.unpin_swa(a[1:2])
    pool.unref_pages(b)
    pool.unref_pages(a)                 # request retires
    assert pool.num_free_pages == 15    # page a[0] survives through the tree's reference
    pool.unref_pages(a[:1])
    pool.assert_no_leak()
    with pytest.raises(AssertionError):
        pool.unref_pages(a[:1])         # double free is caught
    with pytest.raises(RuntimeError):
        pool.alloc_pages(9)             # more pages than SWA slots
    assert bytes_per_page(ModelConfig.flash(), 256) > 1_000_000


def test_radix_match_insert_split_evict():
    pool = _pool(pages=32, swa=32)
    rc = RadixPrefixCache(pool, 16, window=16, align=16)
    toks = np.arange(100, dtype=np.int32)
    pages = pool.alloc_pages(6)
    pool.pin_swa(pages)                  # the running request's window pins
    canon, node = rc.insert(toks[:96], pages)
    assert canon == pages and rc.metrics["inserted_pages"] == 6
    m = rc.match(toks[:95])
    assert m.length == 80 and m.pages == pages[:5]
    pool.unpin_swa(pages)                # the request moved on: only the tree still pins its tail page
    assert all(pool.has_swa(p) for p in pages) and pool.runtime_swa_counters()["swa_slots_reclaimable"] == 5
    assert rc.match(toks[:95]).length == 80  # unpinned window rows are still there: the hit resumes on them
    assert pool.reclaim_swa(100) == 5        # ... until other pages need the slots
    assert [pool.has_swa(p) for p in pages] == [False] * 5 + [True]
    assert rc.match(toks[:100]).length == 96
    assert rc.match(toks[:95]).length == 0   # boundary 80 has no live window storage: the hit backs off
    other = np.concatenate([toks[:40], np.full(40, 7, np.int32)])
    m2 = rc.match(other)
    assert m2.raw_length == 32 and m2.length == 0   # split at the page boundary inside the cached run, no window there
    p2 = pool.alloc_pages(3)
    pool.pin_swa(p2)
    rc.insert(other[:80], pages[:2] + p2)
    assert rc.match(other).length == 80
    pool.unpin_swa(p2)
    rc.lock(node)
    before = pool.num_free_pages
    pool.unref_pages(pages)
    pool.unref_pages(p2)
    assert rc.evict(100) == 3           # only the unlocked branch goes
    rc.unlock(node)
    assert rc.evict(100) == 6 and pool.num_free_pages == 32
    pool.assert_no_leak()
    assert first_mismatch(np.array([1, 2, 3], np.int32), np.array([1, 2, 4, 5], np.int32)) == 2


# ---------------------------------------------------------------------------- small pieces
class _Tok:
    eos_token_id = 99

    def batch_decode(self, rows):
        return ["".join({1: "he", 2: "llo", 3: " wor", 4: "ld", 5: "�", 99: "<eos>"}[i] for i in r) for r in rows]


def test_incremental_detokenizer():
    from minisgl.message import DetokenizeMsg

    d = DetokenizeManager(_Tok())
    out = [d.detokenize([DetokenizeMsg(0, t, f, "stop" if f else None)])[0]
           for t, f in ((1, False), (2, False), (5, False), (3, False), (4, False), (99, True))]
    assert "".join(out) == "hello� world" and 0 not in d.state
    assert printable_prefix("ab cd") == "ab " and printable_prefix("x\n") == "x\n" and printable_prefix("中") == "中"


def test_reasoning_states_and_stats():
    assert initial_reasoning_state(None) == ReasoningState.CHAT and initial_reasoning_state("max") == ReasoningState.THINKING
    with pytest.raises(ValueError):
        initial_reasoning_state("low")
    s = advance_reasoning_state(ReasoningState.THINKING, 5, think_end_token_id=5)
    assert s == ReasoningState.ANSWER and advance_reasoning_state(ReasoningState.CHAT, 5, think_end_token_id=5) == ReasoningState.CHAT
    assert effective_reasoning_state(ReasoningState.THINKING, current_input_token_id=5, think_end_token_id=5) == ReasoningState.ANSWER
    t = [0.0]
    st = StatsTracker(10.0, clock=lambda: t[0])
    st.on_prefill(1000)
    st.on_decode(50)
    assert st.maybe_report(1, 2, 0.5) is None
    t[0] = 10.0
    line = st.maybe_report(1, 2, 0.5)
    assert "prompt 100.0 tok/s" in line and "generation 5.0 tok/s" in line and "KV 50.0%" in line


def test_graph_runner_selects_bucket_and_context_class_without_a_gpu():
    """The replay decision of the graph runner, built with object.__new__ (no capture): which decode batches have a
    captured graph, which bucket they are padded to, which context class they replay, and the status counters."""
    from types import SimpleNamespace

    from minisgl.engine.graph import GraphRunner

    class FakeGraph:
        def __init__(self):
            self.n = 0

        def replay(self):
            self.n += 1

    r = object.__new__(GraphRunner)
    r.buckets, r.classes = [1, 2, 4, 8], [2048, 32768, 1 << 20]
    r.capture_status = {"captured": 12, "replays": 0, "eager_decode": 0, "unsupported_bs": 0, "context_overflow": 0}
    r.graphs = {(b, c): FakeGraph() for b in r.buckets for c in range(3)}
    r.logits = {k: f"logits{k}" for k in r.graphs}
    r.launches = {k: 100 + k[0] for k in r.graphs}
    copies = []
    r.buffer = SimpleNamespace(copy_from=lambda batch, bs: copies.append(bs), next_tokens=torch.arange(8))

    def batch(size, ctx, phase="decode", padded=None):
        n = padded if padded is not None else size
        return SimpleNamespace(is_decode=phase == "decode", size=size, max_context=ctx,
                               positions=torch.zeros(n, dtype=torch.int32))

    assert [r.padded_size(n) for n in (1, 3, 5, 8, 9)] == [1, 4, 8, 8, 9]
    assert [r._class_of(c) for c in (1, 2048, 2049, 32768, 1 << 20, (1 << 20) + 1)] == [0, 0, 1, 1, 2, None]
    assert not r.can_replay(batch(4, 100, phase="prefill"))
    assert not r.can_replay(batch(9, 100)) and r.capture_status["unsupported_bs"] == 1
    assert not r.can_replay(batch(4, (1 << 20) + 1)) and r.capture_status["context_overflow"] == 1
    b = batch(3, 5000, padded=4)
    assert r.can_replay(b)
    from minisgl.ops import native

    n0 = native.launch_count()
    logits, toks = r.replay(b)
    assert logits == "logits(4, 1)" and toks.tolist() == [0, 1, 2, 3] and r.graphs[(4, 1)].n == 1 and copies == [4]
    assert native.launch_count() - n0 == 104 and r.capture_status["replays"] == 1
    with pytest.raises(AssertionError, match="padded"):
        r.replay(batch(3, 5000))                      # not padded to its bucket
    with pytest.raises(RuntimeError, match="no captured graph"):
        r.replay(batch(9, 100, padded=9))
