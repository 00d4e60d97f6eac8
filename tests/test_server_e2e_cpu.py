"""The whole serving stack as processes, on CPU: ``python -m minisgl --device cpu`` on a synthetic checkpoint (tiny
model, word-level tokenizer written to the same folder) spawns the scheduler and the detokenizer under the
supervisor; the test talks to it over HTTP like an OpenAI client -- model list, a completion, a streamed completion,
a rejected parameter -- and stops it with SIGINT.  With ``--tp-size 2`` two scheduler ranks run (gloo collectives,
rank 0 republishing the requests to rank 1)."""
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.error
import urllib.request

import pytest

from minisgl.models import synth
from minisgl.models.config import ModelConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write_tokenizer(folder: str, vocab_size: int) -> None:
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    special = ["<s>", "</s>", "<unk>", "<think>", "</think>"]
    vocab = {t: i for i, t in enumerate(special)}
    for i in range(len(special), vocab_size):
        vocab[f"w{i}"] = i
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    fast.chat_template = ("{% for m in messages %}{{ m['role'] }} {{ m['content'] }} {% endfor %}"
                          "{% if add_generation_prompt %}assistant{% endif %}")
    fast.save_pretrained(folder)
    # the checkpoint's own chat formatter (thinking requests open the reasoning block)
    os.makedirs(os.path.join(folder, "encoding"), exist_ok=True)
    with open(os.path.join(folder, "encoding", "encoding_dsv4.py"), "w") as f:
        f.write("def encode_messages(messages, thinking_mode, reasoning_effort):\n"
                "    text = ' '.join(m['content'] for m in messages)\n"
                "    return text + (' <think>' if thinking_mode == 'thinking' else '')\n")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _http(url, body=None, timeout=120):
    req = urllib.request.Request(url, data=None if body is None else json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.status, r.read().decode()
    except urllib.error.HTTPError as e:
        return e.code, e.read().decode()


@pytest.fixture(scope="module", params=[1, 2], ids=["tp1", "tp2"])
def server(request, tmp_path_factory):
    cfg = ModelConfig.tiny()
    folder = str(tmp_path_factory.mktemp("model"))
    synth.write_checkpoint(cfg, folder, seed=11)
    _write_tokenizer(folder, cfg.vocab_size)
    port = _free_port()
    log = open(os.path.join(folder, "server.log"), "w")
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), LOG_LEVEL="WARNING")
    if request.param == 2:  # the two-rank server also runs the non-overlapped scheduler loop
        env["MINISGL_DISABLE_OVERLAP_SCHEDULING"] = "1"
    proc = subprocess.Popen(
        [sys.executable, "-m", "minisgl", "--model", folder, "--device", "cpu", "--port", str(port), "--page-size", "16",
         "--num-pages", "64", "--max-running-requests", "4", "--context-length", "512", "--served-model-name", "tiny",
         "--disable-log-stats", "--tp-size", str(request.param)]
        + (["--enable-reasoning-sampler-contract"] if request.param == 1 else []), cwd=ROOT, env=env, stdout=log, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"
    deadline = time.time() + 180
    up = False
    while time.time() < deadline and proc.poll() is None:
        try:
            if _http(base + "/v1/models", timeout=2)[0] == 200:
                up = True
                break
        except Exception:
            time.sleep(0.5)
    if not up:
        proc.kill()
        log.close()
        pytest.fail("server did not come up:\n" + open(os.path.join(folder, "server.log")).read()[-3000:])
    yield base, proc, folder
    if proc.poll() is None:
        proc.send_signal(signal.SIGINT)
        try:
            proc.wait(60)
        except subprocess.TimeoutExpired:
            proc.kill()
    log.close()


def test_models_completion_stream_and_errors(server):
    base, proc, folder = server
    code, body = _http(base + "/v1/models")
    assert code == 200 and "tiny" in [m["id"] for m in json.loads(body)["data"]]
    req = {"model": "tiny", "messages": [{"role": "user", "content": "w10 w11 w12 w13"}], "max_tokens": 6,
           "temperature": 0}
    code, body = _http(base + "/v1/chat/completions", req)
    assert code == 200, body
    out = json.loads(body)
    choice = out["choices"][0]
    assert choice["finish_reason"] in ("length", "stop") and isinstance(choice["message"]["content"], str)
    assert out["usage"]["completion_tokens"] <= 6 and out["usage"]["prompt_tokens"] == 4
    first = choice["message"]["content"]
    # greedy decoding of the same prompt is repeatable through the whole stack (and hits the prefix cache path)
    assert json.loads(_http(base + "/v1/chat/completions", req)[1])["choices"][0]["message"]["content"] == first
    # streamed: the chunks spell the same text and end with [DONE]
    code, body = _http(base + "/v1/chat/completions", dict(req, stream=True, stream_options={"include_usage": True}))
    assert code == 200
    events = [l[6:] for l in body.splitlines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    text = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c.get("choices"))
    assert text == first
    assert any(c.get("usage") for c in chunks)
    # an unsupported parameter and an unknown model are refused in OpenAI's error shape
    code, body = _http(base + "/v1/chat/completions", dict(req, n=2))
    assert code == 400 and json.loads(body)["error"]["param"] == "n"
    code, body = _http(base + "/v1/chat/completions", dict(req, model="other"))
    assert code == 404
    assert proc.poll() is None


def test_thinking_request_returns_reasoning_content(server):
    """reasoning_effort: the prompt goes through the checkpoint's formatter, the request starts in the THINKING state
    (with the sampler contract on: <think> never sampled, EOS masked while thinking) and what it generates before a
    closing delimiter is returned as reasoning_content."""
    base, proc, _ = server
    req = {"model": "tiny", "messages": [{"role": "user", "content": "w30 w31 w32"}], "max_tokens": 6,
           "temperature": 0.8, "reasoning_effort": "high"}
    code, body = _http(base + "/v1/chat/completions", req)
    assert code == 200, body
    msg = json.loads(body)["choices"][0]["message"]
    assert "reasoning_content" in msg and isinstance(msg["content"], str)
    words = (msg["reasoning_content"] + " " + msg["content"]).split()
    assert 1 <= len(words) <= 6 and "<think>" not in words and "</s>" not in msg["reasoning_content"].split()
    assert json.loads(body)["usage"]["prompt_tokens"] == 4          # three words + the opening delimiter
    plain = json.loads(_http(base + "/v1/chat/completions", dict(req, reasoning_effort="none"))[1])
    assert "reasoning_content" not in plain["choices"][0]["message"]
    assert proc.poll() is None


def test_online_benchmark_client_measures_the_running_server(server, capsys):
    """The public online benchmark (async streaming client, per-token timestamps) against the live server."""
    import asyncio

    from minisgl.benchmark import client as C
    from minisgl.benchmark.online import bench_simple

    base, proc, _ = server
    items = [C.TraceItem(0.05 * i, " ".join(f"w{40 + i + k}" for k in range(10)), 5) for i in range(5)]
    s = asyncio.run(C.benchmark_trace(base, "tiny", items))
    assert s["requests"] == 5 and s["failed"] == 0
    assert s["ttft"]["p50"] > 0 and s["tpot"]["p50"] > 0 and s["e2e"]["max"] >= s["ttft"]["max"]
    assert s["output_tok_s"] > 0 and s["req_s"] > 0
    bad = asyncio.run(C.benchmark_trace(base, "no-such-model", items[:2]))
    assert bad["failed"] == 2
    bench_simple.main(["--url", base, "--model", "tiny", "--batch", "3", "--input-words", "8", "--output-len", "4"])
    out = json.loads(capsys.readouterr().out)
    assert out["requests"] == 3 and out["failed"] == 0
    assert proc.poll() is None


def test_concurrent_requests_are_all_answered(server):
    import threading

    base, proc, _ = server
    results = {}

    def one(i):
        req = {"model": "tiny", "messages": [{"role": "user", "content": " ".join(f"w{20 + i * 7 + k}" for k in range(12))}],
               "max_tokens": 8, "temperature": 0}
        results[i] = _http(base + "/v1/chat/completions", req)

    threads = [threading.Thread(target=one, args=(i,)) for i in range(6)]   # more than the 4 request slots
    for t in threads:
        t.start()
    for t in threads:
        t.join(180)
    assert sorted(results) == list(range(6))
    for code, body in results.values():
        assert code == 200 and json.loads(body)["usage"]["completion_tokens"] <= 8
    assert proc.poll() is None


def test_zz_a_dead_backend_process_turns_the_api_unavailable(server):
    """Failure detection, host side: one backend child is killed (exact pid, SIGKILL); the health watcher notices
    within seconds, new requests get 503 ``backend_unavailable`` instead of hanging, and the API process survives to
    say so.  Runs last on each server instance."""
    import psutil

    base, proc, _ = server
    kids = [c for c in psutil.Process(proc.pid).children(recursive=True)
            if "resource_tracker" not in " ".join(c.cmdline())]
    assert kids, "the server has backend children"
    victim = max(kids, key=lambda c: c.memory_info().rss)      # a scheduler rank (it holds the weights)
    victim.kill()
    req = {"model": "tiny", "messages": [{"role": "user", "content": "w10 w11"}], "max_tokens": 3, "temperature": 0}
    deadline, code, body = time.time() + 30, None, ""
    while time.time() < deadline:
        code, body = _http(base + "/v1/chat/completions", req, timeout=20)
        if code == 503:
            break
        time.sleep(0.5)
    assert code == 503 and json.loads(body)["error"]["code"] == "backend_unavailable", (code, body[:300])
    assert proc.poll() is None and _http(base + "/v1/models")[0] == 200


def test_shell_mode_chats_over_stdin(tmp_path):
    """``--shell-mode``: the same backend processes behind a line-oriented chat on stdin / stdout."""
    cfg = ModelConfig.tiny()
    folder = str(tmp_path / "model")
    synth.write_checkpoint(cfg, folder, seed=11)
    _write_tokenizer(folder, cfg.vocab_size)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), LOG_LEVEL="ERROR",
               MINISGL_SHELL_MAX_TOKENS="5", MINISGL_SHELL_TEMPERATURE="0.0")
    proc = subprocess.run(
        [sys.executable, "-m", "minisgl", "--model", folder, "--device", "cpu", "--shell-mode", "--page-size", "16",
         "--num-pages", "64", "--context-length", "512"],
        cwd=ROOT, env=env, input="w10 w11 w12\n\n/reset\nw20 w21\n/exit\n", capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    out = proc.stdout
    assert "minisgl shell" in out and out.count("> ") >= 4
    answers = [l for l in out.split("> ") if l.strip() and "minisgl shell" not in l]
    words = [w for a in answers for w in a.split()]
    assert 2 <= len(words) <= 10 and all(w.startswith("w") or w.startswith("<") for w in words), out


def test_offline_example_on_two_cpu_ranks(tmp_path):
    """examples/offline_dsv4.py: a chat prompt through ``LLM.generate`` on two tensor-parallel ranks (gloo), with the
    checkpoint's tokenizer and formatter, printing the decoded text from rank 0."""
    cfg = ModelConfig.tiny()
    folder = str(tmp_path / "model")
    synth.write_checkpoint(cfg, folder, seed=11)
    _write_tokenizer(folder, cfg.vocab_size)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), LOG_LEVEL="ERROR")
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "examples", "offline_dsv4.py"), folder, "--tp", "2", "--device", "cpu",
         "--page-size", "16", "--num-pages", "64", "--prompt", "w50 w51 w52", "--max-tokens", "6"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1                                   # only rank 0 prints
    words = lines[0].split()
    assert 1 <= len(words) <= 6 and all(w.startswith(("w", "<")) for w in words)
