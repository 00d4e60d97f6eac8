"""Multi-rank tests: tensor/expert parallel sharding on CPU (gloo, 2 ranks) and the fused NVLink collectives on GPUs."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, extra, port, env_extra=None, timeout=900):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", **(env_extra or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_worker.py")] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    log_dir = os.environ.get("MINISGL_TEST_LOG_DIR")
    if log_dir and os.path.isdir(log_dir):       # keep the workers' complete output (a traceback scrolls out of a tail)
        with open(os.path.join(log_dir, f"tp_worker_n{nproc}.log"), "w") as f:
            f.write(r.stdout + "\n---- stderr ----\n" + r.stderr)
    first_tb = r.stderr.find("Traceback")
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[max(first_tb, 0):][:3000]
    assert r.stdout.count("OK") >= nproc, r.stdout[-2000:]


@pytest.mark.parametrize("mode", ["ep", "tp"])
def test_cpu_two_ranks_match_single_rank(mode):
    _run(2, ["--device", "cpu", "--moe-mode", mode], 29631 if mode == "ep" else 29632)


@pytest.mark.gpu
def test_gpu_fused_collectives_and_tp_model():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    _run(min(n, 8) if n in (2, 4, 8) else 2, ["--device", "cuda", "--moe-mode", "ep"], 29633,
         {"NCCL_NVLS_ENABLE": "0"})
