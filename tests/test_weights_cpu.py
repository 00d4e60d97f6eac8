"""Checkpoint path on CPU: a synthetic DeepSeek-V4 checkpoint (config.json + safetensors in the raw tensor names)
is written to a temporary folder, streamed back through the loader and compared with the tensors the same seed
produces in memory -- single rank, and both tensor-parallel layouts of the routed experts."""
import json
import os

import pytest
import torch

from helpers import MiniRunner
from minisgl.models import synth
from minisgl.models import weight as W
from minisgl.models.config import ModelConfig


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    cfg = ModelConfig.tiny()
    folder = str(tmp_path_factory.mktemp("ckpt"))
    synth.write_checkpoint(cfg, folder, seed=3)
    return cfg, folder


def _same(a, b):
    assert a.keys() == b.keys(), sorted(set(a) ^ set(b))
    for k in a:
        assert a[k].dtype == b[k].dtype and a[k].shape == b[k].shape, k
        assert torch.equal(a[k].view(torch.uint8) if a[k].dtype.itemsize == 1 else a[k],
                           b[k].view(torch.uint8) if b[k].dtype.itemsize == 1 else b[k]), k


def test_config_round_trips_and_other_architectures_are_refused(ckpt):
    cfg, folder = ckpt
    hf = json.load(open(os.path.join(folder, "config.json")))
    assert ModelConfig.from_hf(hf) == cfg
    with pytest.raises(ValueError, match="not supported"):
        ModelConfig.from_hf(dict(hf, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ValueError, match="not supported"):
        ModelConfig.from_hf(dict(hf, model_type="deepseek_v3"))


def test_single_rank_load_equals_in_memory_weights_and_runs(ckpt):
    cfg, folder = ckpt
    seen = []
    loaded = W.load_checkpoint(folder, cfg, "cpu", progress=seen.append)
    assert seen == [f"layer {l}" for l in range(cfg.num_layers)]
    _same(loaded, synth.random_weights(cfg, "cpu", seed=3))
    toks = list(range(5, 45))
    a = MiniRunner(cfg, "cpu", weights=loaded).step([(0, toks)])
    b = MiniRunner(cfg, "cpu", seed=3).step([(0, toks)])
    assert torch.equal(a, b)


@pytest.mark.parametrize("mode", ["tp", "ep"])
def test_two_rank_shards(ckpt, mode):
    cfg, folder = ckpt
    full = W.load_checkpoint(folder, cfg, "cpu")
    parts = [W.load_checkpoint(folder, cfg, "cpu", rank=r, size=2, moe_mode=mode) for r in range(2)]
    for r in range(2):
        _same(parts[r], synth.random_weights(cfg, "cpu", rank=r, size=2, moe_mode=mode, seed=3))
    cat = lambda k, d: torch.cat([parts[0][k], parts[1][k]], d)
    # vocabulary rows, query heads and the output projection's input columns are split; the rest is replicated
    assert torch.equal(cat("head.weight", 0), full["head.weight"])
    assert torch.equal(cat("L0.attn.wq_b.weight", 0).view(torch.uint8), full["L0.attn.wq_b.weight"].view(torch.uint8))
    assert torch.equal(cat("L0.attn.wo_b.weight", 1).view(torch.uint8), full["L0.attn.wo_b.weight"].view(torch.uint8))
    assert torch.equal(cat("L0.attn.sink", 0), full["L0.attn.sink"])
    for k in ("embed.weight", "L0.attn.wqkv_a.weight", "L0.moe.gate.weight", "L0.hc_attn.fn"):
        assert torch.equal(parts[0][k].view(torch.uint8) if parts[0][k].dtype.itemsize == 1 else parts[0][k],
                           full[k].view(torch.uint8) if full[k].dtype.itemsize == 1 else full[k]), k
    e, i2 = cfg.n_routed_experts, full["L0.moe.w13"].shape[1]
    if mode == "ep":  # whole experts, rank r holds experts [r*E/2, (r+1)*E/2)
        assert parts[0]["L0.moe.w13"].shape[0] == e // 2
        assert torch.equal(cat("L0.moe.w13", 0), full["L0.moe.w13"])
        assert torch.equal(cat("L0.moe.w2", 0), full["L0.moe.w2"])
        assert list(W.local_experts(cfg, 1, 2, "ep")) == list(range(e // 2, e))
    else:            # every expert on every rank, intermediate dimension split (gate and up halves separately)
        assert parts[0]["L0.moe.w13"].shape == (e, i2 // 2, full["L0.moe.w13"].shape[2])
        gate = torch.cat([parts[0]["L0.moe.w13"][:, : i2 // 4], parts[1]["L0.moe.w13"][:, : i2 // 4]], 1)
        assert torch.equal(gate, full["L0.moe.w13"][:, : i2 // 2])
        assert torch.equal(cat("L0.moe.w2", 2), full["L0.moe.w2"])


def test_extra_tensors_are_ignored_and_bad_expert_scales_are_refused(ckpt, tmp_path):
    from safetensors.torch import load_file, save_file

    cfg, folder = ckpt
    import shutil

    work = str(tmp_path / "copy")
    shutil.copytree(folder, work)
    # multi-token-prediction weights and layers beyond the configured depth are not part of the served model
    save_file({"mtp.0.emb.weight": torch.zeros(4, 4), f"layers.{cfg.num_layers}.attn_norm.weight": torch.ones(8)},
              os.path.join(work, "model-extra.safetensors"))
    _same(W.load_checkpoint(work, cfg, "cpu"), W.load_checkpoint(folder, cfg, "cpu"))
    # the block-scaled expert kernel takes every e8m0 byte but 255 (NaN); the fp16 operand kernel only 103..142:
    # a scale the selected kernel cannot represent must stop the load, not corrupt the expert
    from minisgl.ops import cuda as C

    f = os.path.join(work, "model-layer000.safetensors")
    t = load_file(f)
    k = "layers.0.ffn.experts.0.w2.scale"
    s = t[k].view(torch.uint8).clone()
    s.view(-1)[0] = 150
    t[k] = s.view(t[k].dtype)
    save_file(t, f)
    assert C.MOE_KERNEL == "mx"
    W.load_checkpoint(work, cfg, "cpu")
    C.MOE_KERNEL = "f16"
    try:
        with pytest.raises(ValueError, match="outside"):
            W.load_checkpoint(work, cfg, "cpu")
    finally:
        C.MOE_KERNEL = "mx"
    s.view(-1)[0] = 255
    t[k] = s.view(t[k].dtype)
    save_file(t, f)
    with pytest.raises(ValueError, match="NaN"):
        W.load_checkpoint(work, cfg, "cpu")


def test_names_and_shard_rules():
    assert W.remap_name("embed.weight") == "model.embed_tokens.weight"
    assert W.remap_name("head.weight") == "lm_head.weight"
    assert W.remap_name("layers.3.attn.wq_a.scale") == "model.layers.3.self_attn.wq_a.weight_scale_inv"
    assert W.remap_name("layers.3.ffn.experts.7.w1.weight") == "model.layers.3.mlp.experts.7.gate_proj.weight"
    assert W.remap_name("layers.3.ffn.experts.7.w2.scale") == "model.layers.3.mlp.experts.7.down_proj.weight_scale_inv"
    assert W.remap_name("layers.3.ffn.gate.bias") == "model.layers.3.mlp.gate.e_score_correction_bias"
    assert W.remap_name("layers.0.ffn.gate.tid2eid") == "model.layers.0.mlp.topk.tid2eid"
    assert W.remap_name("layers.1.ffn_norm.weight") == "model.layers.1.post_attention_layernorm.weight"
    assert W.shard_rows(129280, 7, 8) == (113120, 129280)
    t = torch.arange(24.0).reshape(6, 4)
    assert W.shard_tensor("layers.0.attn.wq_b.weight", t, 1, 2).tolist() == t[3:].tolist()
    assert W.shard_tensor("layers.0.attn.wo_b.weight", t, 1, 2).tolist() == t[:, 2:].tolist()
    assert W.shard_tensor("layers.0.attn.wq_a.weight", t, 1, 2) is t
    assert W.shard_tensor("layers.0.ffn.experts.1.w2.weight", t, 0, 2, "ep") is t
    with pytest.raises(ValueError, match="does not split"):
        W.shard_tensor("layers.0.attn.wq_b.weight", t[:5], 0, 2)
