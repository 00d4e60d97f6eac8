"""CPU oracle model: chunked prefill and token-by-token decode must reproduce a single-shot prefill."""
import torch

from helpers import MiniRunner
from minisgl.models.config import ModelConfig


def _prompt(n, seed=0, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def test_single_shot_vs_chunked_vs_decode():
    cfg = ModelConfig.tiny()
    toks = _prompt(150)
    a = MiniRunner(cfg)
    la = a.step([(0, toks)])
    b = MiniRunner(cfg)
    b.step([(0, toks[:37])])
    b.step([(0, toks[37:100])])
    lb = b.step([(0, toks[100:])])
    assert torch.equal(la.argmax(-1), lb.argmax(-1))
    assert torch.allclose(la, lb, atol=4e-2, rtol=4e-2), (la - lb).abs().max()
    c = MiniRunner(cfg)
    c.step([(0, toks[:140])])
    lc = None
    for t in toks[140:]:
        lc = c.step([(0, [t])])
    assert torch.equal(la.argmax(-1), lc.argmax(-1))
    assert torch.allclose(la, lc, atol=4e-2, rtol=4e-2), (la - lc).abs().max()


def test_batched_requests_are_independent():
    cfg = ModelConfig.tiny()
    t0, t1 = _prompt(70, 1), _prompt(45, 2)
    a = MiniRunner(cfg)
    l0 = a.step([(0, t0)])
    l1 = a.step([(1, t1)])
    b = MiniRunner(cfg)
    lb = b.step([(0, t0), (1, t1)])
    assert torch.allclose(lb[0], l0[0], atol=4e-2, rtol=4e-2)
    assert torch.allclose(lb[1], l1[0], atol=4e-2, rtol=4e-2)


def test_cache_state_matches_between_chunked_and_single_shot():
    cfg = ModelConfig.tiny()
    toks = _prompt(150, 3)
    a = MiniRunner(cfg)
    a.step([(0, toks)])
    b = MiniRunner(cfg)
    for i in range(0, 150, 29):
        b.step([(0, toks[i:i + 29])])
    n4 = 150 // 4
    assert torch.allclose(a.pool.c4[0][:n4].float(), b.pool.c4[0][:n4].float(), atol=3e-2)
    assert torch.allclose(a.pool.c128[0][:1].float(), b.pool.c128[0][:1].float(), atol=3e-2)
    same = (a.pool.idx_vals[0][:n4] == b.pool.idx_vals[0][:n4]).float().mean()
    assert same > 0.9, same
    close = ((a.pool.swa[1][:150].float() - b.pool.swa[1][:150].float()).abs() < 5e-2).float().mean()
    assert close > 0.98, close  # an e4m3 rounding flip in the QAT step moves a value by a full fp8 ulp


def test_checked_run_audits_gathered_indices(monkeypatch):
    """MINISGL_DEBUG_BOUNDS=1: a forward with valid indices passes the audit (and gives the same logits); a token id
    outside the vocabulary is refused before anything is gathered with it."""
    import pytest

    cfg = ModelConfig.tiny()
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(3)).tolist()
    plain = MiniRunner(cfg, "cpu", seed=5).step([(0, toks)])
    monkeypatch.setenv("MINISGL_DEBUG_BOUNDS", "1")
    checked = MiniRunner(cfg, "cpu", seed=5)
    assert checked.model._debug_bounds
    assert torch.equal(checked.step([(0, toks)]), plain)
    with pytest.raises(IndexError, match="input_ids"):
        checked.step([(1, [cfg.vocab_size + 7])])
