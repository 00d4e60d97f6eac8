"""Pins this repository's PyTorch operator oracle (minisgl.ops.ref / minisgl.ops.quant -- the reference every CUDA
kernel test compares against) to the reference project's own torch oracle, op by op.

The reference ships pure-PyTorch restatements of its kernels in debug/dsv4/kernel/deepseek_v4_reference.py.  They
are run in a child process (tests/ref_oracle_worker.py) from a reference checkout found in $DSV4_REFERENCE_DIR or in
a directory named ``reference`` next to this repository; without one the tests are skipped.

One operator is deliberately not compared in its overlap form: that file's ratio-4 compressor pools the left and
right halves of the SAME four tokens, whereas the reference's production kernel (and the model it serves) pools the
left halves of the previous four tokens with the right halves of the current four
(python/minisgl/kernel/triton/deepseek_v4.py:2440-2476).  This repository follows the production kernel; the
non-overlap (ratio 128) compressor is compared.
"""
import os
import subprocess
import sys

import pytest
import torch

from minisgl.ops import quant, ref
from minisgl.ops.ref import RopeSpec

HERE = os.path.dirname(os.path.abspath(__file__))


def _reference_dir():
    cands = [os.environ.get("DSV4_REFERENCE_DIR", ""), os.path.join(HERE, "..", "..", "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "debug", "dsv4", "kernel", "deepseek_v4_reference.py")):
            return os.path.abspath(c)
    return None


@pytest.fixture(scope="module")
def golden(tmp_path_factory):
    root = _reference_dir()
    if root is None:
        pytest.skip("no reference checkout (set DSV4_REFERENCE_DIR)")
    out = tmp_path_factory.mktemp("oracle") / "golden.pt"
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    r = subprocess.run([sys.executable, os.path.join(HERE, "ref_oracle_worker.py"), root, str(out)],
                       capture_output=True, text=True, timeout=900, cwd=str(out.parent), env=env)
    if r.returncode != 0:
        pytest.skip("the reference oracle did not run here: " + (r.stderr.strip().splitlines() or ["?"])[-1][:200])
    return torch.load(out, weights_only=False)


def test_fp8_activation_quant_is_bit_exact(golden):
    g = golden["fp8_act"]
    assert torch.equal(quant.fp8_fake_quant(g["x"]).to(torch.bfloat16), g["y"])
    q, s = quant.fp8_act_quant(g["x"])
    assert torch.equal((q.float().view(10, 4, 128) * s[:, :, None]).view(10, 512).to(torch.bfloat16), g["y"])


def test_fp4_dequant_is_bit_exact(golden):
    g = golden["fp4"]
    assert torch.equal(quant.fp4_dequant(g["packed"], g["codes"], dtype=torch.float32), g["w"])


def test_c128_compressor_pooling(golden):
    g = golden["compress128"]
    x, w, ape = g["x"], g["w"], g["ape"]
    t, d, ps = x.shape[0], ape.shape[1], 128
    proj = (x @ w.t()).float()
    pos = torch.arange(t, dtype=torch.int32)
    slots = torch.zeros(t, dtype=torch.int32)
    table = torch.arange(512, dtype=torch.int32)[None, :]
    ring = torch.zeros(128, 2 * d)
    mine = ref.compress_pool(proj, pos, slots, 128, d, ape, ring, None, table, ps)
    ends = [i for i in range(t) if (i + 1) % 128 == 0]
    assert g["pooled"].shape[0] == len(ends) == 2
    torch.testing.assert_close(mine[ends], g["pooled"].float(), rtol=1e-5, atol=1e-6)
    assert float(mine[[i for i in range(t) if i not in ends]].abs().max()) == 0.0


def test_rotary_tail_plain_and_scaled(golden):
    g = golden["rope"]
    specs = {"plain": RopeSpec.make(64, 10000.0), "yarn": RopeSpec.make(64, 160000.0, 65536, 16.0, 32, 1)}
    for (name, inv), want in g["y"].items():
        got = ref.rope_tail(g["x"].clone(), g["pos"].to(torch.int32), specs[name], inverse=inv)
        # The two restatements build the inverse frequencies differently (exp(-k log b) here, as the reference's
        # kernel does, against 1 / b**k there): they differ by an fp32 rounding, i.e. by ~1e-7 * position radians.
        err = (got.float() - want.float()).abs().amax(dim=(1, 2))
        tol = 2e-5 + g["pos"].float() * 1.2e-7
        assert bool((err <= tol).all()), (err, tol)
        assert torch.equal(got[..., :32], g["x"][..., :32])        # the head of each vector is left alone


def test_indexer_logits(golden):
    g = golden["indexer"]
    ps, lens, table = g["ps"], g["lens"], g["table"]
    jmax = int(lens.max())
    j = torch.arange(jmax)
    rows = table.long()[:, j // ps] * ps + (j % ps)[None, :]
    mine = ref.indexer_logits(g["q"], g["w"], g["vals"].view(-1, 128), g["scales"], rows, lens)
    want = g["logits"]
    assert want.shape == mine.shape
    valid = j[None, :] < lens[:, None]
    assert bool(torch.isinf(mine[~valid]).all()) and bool(torch.isinf(want[~valid]).all())
    torch.testing.assert_close(mine[valid], want[valid], rtol=2e-5, atol=1e-4)


def test_hyper_connection_mixes(golden):
    g = golden["hc"]
    y, post, comb = ref.hc_pre(g["x"], g["fn"], g["scale"], g["base"], 20, 1e-6, 1e-6)
    # the reference rounds the mixing weights to bf16 before applying them; this oracle keeps them in fp32
    torch.testing.assert_close(post, g["post"].float(), rtol=8e-3, atol=1e-3)
    torch.testing.assert_close(comb, g["comb"].float(), rtol=8e-3, atol=1e-3)
    torch.testing.assert_close(y.float(), g["y"].float(), rtol=2e-2, atol=2e-2)
    assert float((comb.sum(1) - 1).abs().max()) < 1e-3 and float((comb.sum(2) - 1).abs().max()) < 1e-3
    mixed = ref.hc_post(g["blk"], g["x"], g["post"].float(), g["comb"].float())
    torch.testing.assert_close(mixed.float(), g["mixed"].float(), rtol=2e-2, atol=2e-2)
    head = ref.hc_head(g["x"], g["fn_head"], torch.tensor([1.1]), g["base_head"], 1e-6, 1e-6)
    torch.testing.assert_close(head.float(), g["head"].float(), rtol=2e-2, atol=2e-2)


def test_rms_norm(golden):
    g = golden["rms"]
    got = ref.rms_norm(g["x"], g["w"], 1e-6)
    torch.testing.assert_close(got.float(), g["y"].float(), rtol=8e-3, atol=1e-3)


def test_sparse_attention_with_sink(golden):
    g = golden["attention"]
    n = max(len(c) for c in g["ctx"])
    rows = torch.full((len(g["ctx"]), n), -1, dtype=torch.int64)
    for i, c in enumerate(g["ctx"]):
        rows[i, : len(c)] = c
    # split every row's context between the "compressed" and the "window" argument: the union is what counts
    mine = ref.sparse_attention(g["q"], g["cache"], rows[:, : n // 2], g["cache"], rows[:, n // 2:], g["sink"],
                                g["q"].shape[-1] ** -0.5)
    torch.testing.assert_close(mine.float(), g["o"].float(), rtol=8e-3, atol=4e-3)


def test_swiglu_with_clamp(golden):
    g = golden["swiglu"]
    gu = torch.cat([g["gate"], g["up"]], dim=-1)
    torch.testing.assert_close(ref.silu_mul_clamp(gu, 7.0).float(), g["y7"].float(), rtol=8e-3, atol=1e-3)
    torch.testing.assert_close(ref.silu_mul_clamp(gu, None).float(), g["y0"].float(), rtol=8e-3, atol=1e-3)
