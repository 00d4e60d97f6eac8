"""The benchmark tooling itself, on CPU: latency statistics, trace readers, exact-length prompt generation, the
launch-list summariser, the chat formatter hook of the tokenizer, and that every public benchmark script imports
and parses its arguments."""
import importlib
import json
import math

import pytest

from minisgl.benchmark import client as C
from minisgl.benchmark import ncu_summary as N


def test_percentiles_and_latency_summary():
    assert C.percentile([], 50) != C.percentile([], 50)  # NaN
    assert C.percentile([4.0, 1.0, 3.0, 2.0], 50) == 2.5 and C.percentile([1.0, 2.0], 100) == 2.0
    a = C.RequestResult(tics=[1.0, 1.1, 1.2, 1.3], t_start=0.5)
    b = C.RequestResult(tics=[2.0], t_start=1.0)
    bad = C.RequestResult(ok=False)
    assert a.ttft == pytest.approx(0.5) and a.tpot == pytest.approx(0.1) and a.e2e == pytest.approx(0.8)
    assert b.tpot is None and bad.ttft is None
    s = C.summarize([a, b, bad], wall_s=2.0)
    assert s["requests"] == 3 and s["failed"] == 1
    assert s["ttft"]["avg"] == pytest.approx(0.75) and s["ttft"]["max"] == pytest.approx(1.0)
    assert s["tpot"]["p50"] == pytest.approx(0.1)       # the one-token request has no inter-token time
    assert s["output_tok_s"] == pytest.approx(2.5) and s["req_s"] == pytest.approx(1.0)


def test_trace_readers_and_scaling(tmp_path):
    p = tmp_path / "trace.jsonl"
    p.write_text("\n".join(json.dumps(d) for d in [
        {"chat_id": 1, "timestamp": 100.0, "input_length": 12, "output_length": 5},
        {"chat_id": 2, "timestamp": 101.5, "input_length": 0, "output_length": 0},
        {"chat_id": 3, "timestamp": 104.0, "input_length": 7, "output_length": 9}]))
    q = C.read_qwen_trace(str(p))
    assert [i.arrival_s for i in q] == [0.0, 1.5, 4.0] and [i.output_len for i in q] == [5, 1, 9]
    assert q[0].prompt.count("x") == 12 and q[1].prompt.count("x") == 1
    assert len(C.read_qwen_trace(str(p), limit=2)) == 2
    m = C.read_mooncake_trace(str(p))                  # same columns, timestamps in milliseconds
    assert [i.arrival_s for i in m] == [0.0, 0.0015, 0.004]
    fast = C.scale_traces(q, 4.0)
    assert [i.arrival_s for i in fast] == [0.0, 0.375, 1.0] and fast[2].output_len == 9 and q[2].arrival_s == 4.0


def test_synthetic_chat_trace_is_reproducible_and_within_bounds():
    a = C.synthetic_chat_trace(200, rate=8.0, seed=1)
    b = C.synthetic_chat_trace(200, rate=8.0, seed=1)
    assert [(i.arrival_s, i.output_len, i.input_len) for i in a] == [(i.arrival_s, i.output_len, i.input_len) for i in b]
    assert all(x.arrival_s < y.arrival_s for x, y in zip(a, a[1:]))
    assert all(16 <= i.input_len <= 16384 and 1 <= i.output_len <= 4096 for i in a)
    assert 200 / a[-1].arrival_s == pytest.approx(8.0, rel=0.3)
    from collections import Counter

    most_common_head = Counter(i.prompt[:40] for i in a).most_common(1)[0][1]
    assert 0.15 * 200 < most_common_head < 0.45 * 200     # about 30 % of the requests open with the common prefix


class _WordTok:
    """A tokenizer in which random ids are not the canonical encoding of their own text: an id that is a multiple of
    7 decodes to two words, which encode back to two other ids (as merged tokens do after a round trip)."""

    vocab_size = 50000

    def decode(self, ids):
        return " ".join(f"t{i + 1} t{i + 2}" if i % 7 == 0 else f"t{i}" for i in ids)

    def encode(self, text, add_special_tokens=False):
        return [int(w[1:]) for w in text.split()]


def test_generate_prompt_hits_the_exact_token_count():
    tok = _WordTok()
    for n in (1, 17, 300):
        assert len(tok.encode(C.generate_prompt(tok, n, seed=n))) == n


def test_launch_list_summary(tmp_path):
    rows = [("void <unnamed>::embed_kernel(int const*)", "(4, 1, 1)", 2000), ("void foo<1>(float*)", "(8, 1, 1)", 9000),
            ("void <unnamed>::embed_kernel(int const*)", "(4, 1, 1)", 1000), ("void foo<1>(float*)", "(8, 1, 1)", 3000),
            ("void foo<1>(float*)", "(8, 1, 1)", 5000), ("void bar(int)", "(1, 1, 1)", 1000)]
    p = tmp_path / "launches.csv"
    with open(p, "w") as f:
        f.write("==PROF== Connected to process 1\n")
        f.write('"ID","Process ID","Kernel Name","Grid Size","Metric Name","Metric Unit","Metric Value"\n')
        for i, (n, g, v) in enumerate(rows):
            f.write(f'"{i}","1","{n}","{g}","gpu__time_duration.sum","ns","{v:,}"\n')
            f.write(f'"{i}","1","{n}","{g}","other__metric","ns","1"\n')
    launches = N.read_launches(str(p))
    assert len(launches) == 6 and launches[1][2] == 9000.0
    step = N.last_step(launches)                      # from the LAST embed launch on
    assert len(step) == 4 and N.last_step(launches, "nothing") == launches
    agg = N.aggregate(step)
    assert list(agg.items())[0] == (("foo<1>", "(8, 1, 1)"), (2, 8000.0))
    assert agg[("embed_kernel", "(4, 1, 1)")] == (1, 1000.0)
    text = N.render(step)
    assert "kernels in last step 4 total us 10.0" in text and " 80.0%" in text
    assert N.main([str(p)]) == 0 and N.main([]) == 2


def test_chat_formatter_from_the_model_folder(tmp_path):
    from types import SimpleNamespace

    from minisgl.tokenizer.tokenize import TokenizeManager, load_dsv4_chat_formatter

    tok = SimpleNamespace(encode=lambda s: [ord(c) for c in s],
                          apply_chat_template=lambda m, tokenize, add_generation_prompt: "T:" + m[-1]["content"])
    msgs = [{"role": "user", "content": "hi"}]
    assert load_dsv4_chat_formatter(str(tmp_path)) is None
    plain = TokenizeManager(tok, str(tmp_path))
    assert plain.render("raw text", None) == "raw text" and plain.render(msgs, None) == "T:hi"
    with pytest.raises(ValueError, match="reasoning_effort"):
        plain.render(msgs, "high")
    enc = tmp_path / "encoding"
    enc.mkdir()
    (enc / "encoding_dsv4.py").write_text(
        "def encode_messages(messages, thinking_mode, reasoning_effort):\n"
        "    return f\"<{thinking_mode}|{reasoning_effort}>\" + messages[-1]['content']\n")
    tm = TokenizeManager(tok, str(tmp_path))
    assert tm.render(msgs, None) == "<chat|None>hi" and tm.render(msgs, "max") == "<thinking|max>hi"
    ids = tm.tokenize([SimpleNamespace(text=msgs, reasoning_effort="high"), SimpleNamespace(text="ab", reasoning_effort=None)])
    assert ids[0].tolist() == [ord(c) for c in "<thinking|high>hi"] and ids[1].tolist() == [97, 98]


@pytest.mark.parametrize("mod", ["offline.bench", "offline.bench_wildchat", "online.bench_simple", "online.bench_qwen",
                                 "perf_matrix", "scheduler_sim", "decode_step", "moe_gemm", "ops", "collectives",
                                 "online_trace", "coverage_run"])
def test_public_benchmark_scripts_import_and_describe_their_arguments(mod, capsys):
    m = importlib.import_module("minisgl.benchmark." + mod)
    assert callable(m.main) and (m.__doc__ or "").strip()
    with pytest.raises(SystemExit) as e:
        m.main(["--help"])
    assert e.value.code == 0 and "usage" in capsys.readouterr().out.lower()


def test_root_bench_and_example_compile():
    import os
    import py_compile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for f in ("bench.py", "__graft_entry__.py", os.path.join("examples", "offline_dsv4.py")):
        py_compile.compile(os.path.join(root, f), doraise=True)
    assert not math.isnan(C.percentile([1.0], 99))


def test_generate_prompt_never_exceeds_the_count_with_an_unstable_tokenizer():
    class Growing(_WordTok):                               # multiples of 7 double on every round trip: no fixed point
        def decode(self, ids):
            return " ".join(f"t{i} t{i}" if i % 7 == 0 else f"t{i}" for i in ids)

    tok = Growing()
    for n in (17, 64):
        assert len(tok.encode(C.generate_prompt(tok, n, seed=n))) <= n


def test_online_trace_runs_timed_arrivals_through_the_engine():
    """Poisson arrivals in wall-clock time on the tiny CPU model: every request finishes with its full output, the
    shared prefix gives radix hits, latencies come out ordered (p50 <= p99), and the perf-matrix harness reports its
    per-scenario figures and the memory ledger."""
    from minisgl.benchmark import online_trace, perf_matrix

    res = online_trace.main(["--tiny", "--device", "cpu", "--page-size", "16", "--num-pages", "512", "--max-running",
                             "8", "--requests", "10", "--rates", "40", "--prompt-median", "60", "--output-median", "6",
                             "--max-prompt", "300", "--max-output", "12"])
    r = res[0]
    assert r["requests"] == r["finished"] == 10 and r["output_tokens"] > 10
    assert r["ttft_s"]["p50"] <= r["ttft_s"]["p99"] and r["tpot_ms"]["p50"] <= r["tpot_ms"]["p99"]
    trace = online_trace.token_trace(200, 8.0, 1000, seed=3)
    gaps = [b[0] - a[0] for a, b in zip(trace, trace[1:])]
    assert all(g >= 0 for g in gaps) and 0.08 < sum(gaps) / len(gaps) < 0.2          # mean gap ~ 1 / rate
    assert all(16 <= len(t[1]) <= 16384 and 1 <= t[2] <= 4096 for t in trace)
    out = perf_matrix.main(["--tiny", "--device", "cpu", "--page-size", "16", "--num-pages", "256", "--max-running", "8",
                            "--scale", "0.05", "--scenarios", "P1K_M8", "--ledger"])
    assert out[0]["requests"] == 8 and out[0]["ledger"]["kv_plan"]["num_pages"] == 256
