"""The harnesses that need no GPU: static audit + census, scheduler policy simulation, scenario catalogue."""
from minisgl.benchmark import audit, perf_matrix, scheduler_sim


def test_static_audit_is_clean():
    rep = audit.audit()
    assert rep["violations"] == [], rep["violations"]
    assert rep["num_kernels"] >= 25 and rep["num_exports"] >= 30
    assert rep["lines"]["tests"] > 500


def test_scheduler_sim_long_prefill_does_not_starve_short_prompts():
    res = scheduler_sim.simulate(scheduler_sim.scenario("long_prefill"))
    done = res["prefill_done_step"]
    assert all(done[u] <= 1 for u in range(1, 16))       # short prompts finish in the first prefill forward(s)
    assert done[0] > 5                                     # the 64 K prompt takes many chunks
    assert res["inter_token_ms"]["max"] < 60               # decodes keep running in between (2 048-token chunks)
    # never two prefills back to back while decodes are runnable (the short requests decode for 32 tokens)
    assert "PP" not in res["first_steps"][1:30]


def test_scheduler_sim_mixed_policy_bounds_decode_gaps():
    calm = scheduler_sim.simulate(scheduler_sim.scenario("mixed"), max_consecutive_decode=4)
    eager = scheduler_sim.simulate(scheduler_sim.scenario("mixed"), max_consecutive_decode=1)
    assert eager["ttft_ms"]["p99"] <= calm["ttft_ms"]["p99"]       # more prefill turns -> earlier first tokens
    assert calm["inter_token_ms"]["p99"] < 40


def test_perf_matrix_catalogue():
    cat = perf_matrix.catalogue()
    assert {"P1K_M128", "P4K_M256", "MIXED_ARRIVAL", "LONG_RESIDENT_64K", "PRESSURE_1M"} <= set(cat)
    assert len(cat["P1K_M128"].prompt_lens) == 128 and cat["P1K_M128"].prompt_lens[0] == 1024
    assert sum(cat["PRESSURE_1M"].prompt_lens) == 1 << 20


def test_perf_matrix_runs_scenarios_on_the_cpu_model(capsys):
    """Scaled-down scenarios through the instrumented offline engine (tiny model, PyTorch oracle): identical prompts
    arriving over time hit the prefix cache; one long prompt beside short ones is chunked while the short ones finish."""
    common = ["--tiny", "--device", "cpu", "--page-size", "16", "--num-pages", "640", "--max-running", "32"]
    sp = perf_matrix.main(common + ["--scale", "0.125", "--scenarios", "SHARED_PREFIX"])[0]
    assert sp["requests"] == 32 and sp["output_tokens"] == 32 * 8
    # 256-token prompts: every arrival after the first prompt was cached resumes at the 128-token boundary
    assert sp["prefix"]["hit_tokens"] >= 128 * 16 and sp["prefix"]["hit_rate"] > 0.25
    lr = perf_matrix.main(common + ["--scale", "0.0625", "--scenarios", "LONG_RESIDENT_64K"])[0]
    assert lr["requests"] == 32 and lr["prompt_tokens"] == 4096 + 31 * 32 and lr["output_tokens"] == 32 * 8
    assert lr["steps"]["prefill"] >= 1 and lr["steps"]["decode"] >= 7
    assert '"scenario": "SHARED_PREFIX"' in capsys.readouterr().out


def test_offline_benchmarks_run_on_the_cpu_model(tmp_path):
    """The public offline benchmarks (fixed wave; mixed-length prompts with temperature sampling) through
    ``LLM.generate`` on the tiny model."""
    from minisgl.benchmark.offline import bench, bench_wildchat

    cpu = ["--tiny", "--device", "cpu", "--page-size", "16", "--num-pages", "256"]
    res = bench.main(cpu + ["-M", "6", "--input-len", "48", "--output-len", "5"])
    assert res["requests"] == 6 and res["output_tok_s"] > 0 and res["prefix"]["queries"] == 6
    wc = bench_wildchat.main(cpu + ["-n", "8", "--max-tokens", "4", "--max-prompt", "200"])
    assert wc["requests"] == 8 and set(wc["finish_reasons"]) <= {"length", "stop"}
