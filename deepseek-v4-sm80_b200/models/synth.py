"""Random-init weights in the checkpoint's own format.

``make_raw_layer`` / ``make_raw_top`` produce the raw tensors of one layer / of the embedding block under
their checkpoint names; ``random_weights`` pipes them through the same shard-and-merge code as a real
checkpoint (:mod:`minisgl.models.weight`), so every rank of a tensor-parallel group derives its shard from
identical full tensors (the generators are seeded per layer).  ``write_checkpoint`` stores a small model
as ``config.json`` + safetensors for loader tests.  Plays the role of the reference's ``--dummy-weight``
(python/minisgl/engine/engine.py:329-335), but with valid quantised tensors instead of ``randn`` bytes.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..ops import quant
from . import weight as W
from .config import ModelConfig

STD = 0.02


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn(shape, g, device, std=STD):
    return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std


def _fp8(shape, g, device) -> Dict[str, torch.Tensor]:
    q, s = quant.fp8_weight_quant(_randn(shape, g, device))
    return {"weight": q, "scale": s}


def _put(out, prefix, d):
    for k, v in d.items():
        out[f"{prefix}.{k}"] = v


def make_raw_top(cfg: ModelConfig, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = _gen(device, seed * 1000003 + 7)
    m, h = cfg.hc_mult, cfg.hidden_size
    return {
        "embed.weight": _randn((cfg.vocab_size, h), g, device).to(torch.bfloat16),
        "head.weight": _randn((cfg.vocab_size, h), g, device).to(torch.bfloat16),
        "norm.weight": torch.ones(h, dtype=torch.bfloat16, device=device),
        "hc_head_fn": _randn((m, m * h), g, device),
        "hc_head_scale": torch.ones(1, dtype=torch.float32, device=device),
        "hc_head_base": torch.zeros(m, dtype=torch.float32, device=device),
    }


def make_raw_layer(cfg: ModelConfig, l: int, device, seed: int = 0, fast_experts: bool = False) -> Dict[str, torch.Tensor]:
    """Raw tensors of layer ``l`` keyed without the ``layers.l.`` prefix.  With ``fast_experts`` the packed FP4
    expert bytes are drawn directly (uniform nibbles, scales 2^-8..2^-6) instead of quantising Gaussians."""
    g = _gen(device, seed * 1000003 + 100 + l)
    h, d, m = cfg.hidden_size, cfg.head_dim, cfg.hc_mult
    out: Dict[str, torch.Tensor] = {}
    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    out["attn_norm.weight"] = ones(h)
    out["ffn_norm.weight"] = ones(h)
    mix = (2 + m) * m
    for k in ("hc_attn", "hc_ffn"):
        out[k + "_fn"] = _randn((mix, m * h), g, device)
        out[k + "_scale"] = torch.ones(3, dtype=torch.float32, device=device)
        out[k + "_base"] = _randn((mix,), g, device, 0.5)
    _put(out, "attn.wq_a", _fp8((cfg.q_lora_rank, h), g, device))
    _put(out, "attn.wkv", _fp8((d, h), g, device))
    _put(out, "attn.wq_b", _fp8((cfg.num_heads * d, cfg.q_lora_rank), g, device))
    _put(out, "attn.wo_a", _fp8((cfg.o_groups * cfg.o_lora_rank, cfg.num_heads * d // cfg.o_groups), g, device))
    _put(out, "attn.wo_b", _fp8((h, cfg.o_groups * cfg.o_lora_rank), g, device))
    out["attn.q_norm.weight"] = ones(cfg.q_lora_rank)
    out["attn.kv_norm.weight"] = ones(d)
    out["attn.attn_sink"] = _randn((cfg.num_heads,), g, device, 1.0)
    ratio = cfg.ratio(l)
    if ratio:
        c = 2 if ratio == 4 else 1
        out["attn.compressor.ape"] = _randn((ratio, c * d), g, device, 0.5)
        out["attn.compressor.wkv.weight"] = _randn((c * d, h), g, device).to(torch.bfloat16)
        out["attn.compressor.wgate.weight"] = _randn((c * d, h), g, device).to(torch.bfloat16)
        out["attn.compressor.norm.weight"] = ones(d)
    if ratio == 4:
        di = cfg.index_head_dim
        _put(out, "attn.indexer.wq_b", _fp8((cfg.index_n_heads * di, cfg.q_lora_rank), g, device))
        out["attn.indexer.weights_proj.weight"] = _randn((cfg.index_n_heads, h), g, device).to(torch.bfloat16)
        out["attn.indexer.compressor.ape"] = _randn((4, 2 * di), g, device, 0.5)
        out["attn.indexer.compressor.wkv.weight"] = _randn((2 * di, h), g, device).to(torch.bfloat16)
        out["attn.indexer.compressor.wgate.weight"] = _randn((2 * di, h), g, device).to(torch.bfloat16)
        out["attn.indexer.compressor.norm.weight"] = ones(di)
    e, inter = cfg.n_routed_experts, cfg.moe_intermediate_size
    out["ffn.gate.weight"] = _randn((e, h), g, device, 0.1).to(torch.bfloat16)
    if l < cfg.n_hash_layers:
        out["ffn.gate.tid2eid"] = _hash_table(cfg, g, device)
    else:
        out["ffn.gate.bias"] = _randn((e,), g, device, 0.01)
    if fast_experts:
        w1 = torch.randint(0, 256, (e, inter, h // 2), generator=g, device=device, dtype=torch.uint8).view(torch.int8)
        w3 = torch.randint(0, 256, (e, inter, h // 2), generator=g, device=device, dtype=torch.uint8).view(torch.int8)
        w2 = torch.randint(0, 256, (e, h, inter // 2), generator=g, device=device, dtype=torch.uint8).view(torch.int8)
        s1 = torch.randint(119, 122, (e, inter, h // 32), generator=g, device=device, dtype=torch.uint8)
        s3 = torch.randint(119, 122, (e, inter, h // 32), generator=g, device=device, dtype=torch.uint8)
        s2 = torch.randint(119, 122, (e, h, inter // 32), generator=g, device=device, dtype=torch.uint8)
    else:
        w1, s1 = quant.fp4_quant(_randn((e, inter, h), g, device))
        w3, s3 = quant.fp4_quant(_randn((e, inter, h), g, device))
        w2, s2 = quant.fp4_quant(_randn((e, h, inter), g, device))
    for i in range(e):
        out[f"ffn.experts.{i}.w1.weight"], out[f"ffn.experts.{i}.w1.scale"] = w1[i], s1[i]
        out[f"ffn.experts.{i}.w3.weight"], out[f"ffn.experts.{i}.w3.scale"] = w3[i], s3[i]
        out[f"ffn.experts.{i}.w2.weight"], out[f"ffn.experts.{i}.w2.scale"] = w2[i], s2[i]
    si = cfg.n_shared_experts * inter
    _put(out, "ffn.shared_experts.w1", _fp8((si, h), g, device))
    _put(out, "ffn.shared_experts.w3", _fp8((si, h), g, device))
    _put(out, "ffn.shared_experts.w2", _fp8((h, si), g, device))
    return out


def _hash_table(cfg: ModelConfig, g, device) -> torch.Tensor:
    """tid2eid [vocab, topk]: distinct experts per token id."""
    k, e = cfg.num_experts_per_tok, cfg.n_routed_experts
    first = torch.randint(0, e, (cfg.vocab_size, 1), generator=g, device=device)
    step = torch.arange(k, device=device)[None, :] * (e // k if e >= k else 1)
    return ((first + step) % e).to(torch.int32)


def random_weights(cfg: ModelConfig, device, rank: int = 0, size: int = 1, moe_mode: str = "tp", seed: int = 0,
                   fast_experts: bool = False, draw_on_host: bool = False) -> Dict[str, torch.Tensor]:
    """Runtime tensors of a random-init model, sharded for (rank, size).  ``draw_on_host``: the raw tensors are drawn
    and quantised on the CPU and only the shards are copied to ``device`` (slow for a full model, but it keeps the
    device's kernel stream free of initialisation kernels -- a small smoke model uses it so that the first launches a
    profiler sees are the model's own)."""
    out: Dict[str, torch.Tensor] = {}
    src = "cpu" if draw_on_host else device
    move = (lambda t: t.to(device)) if draw_on_host else (lambda t: t)
    top = {k: move(W.shard_tensor(k, v, rank, size, moe_mode)) for k, v in make_raw_top(cfg, src, seed).items()}
    out.update(W.build_top(cfg, top))
    experts = set(W.local_experts(cfg, rank, size, moe_mode))
    for l in range(cfg.num_layers):
        raw = make_raw_layer(cfg, l, src, seed, fast_experts)
        sh = {}
        for k, v in raw.items():
            full = f"layers.{l}.{k}"
            m = W._EXPERT.match(full)
            if m is not None and int(m.group(2)) not in experts:
                continue
            sh[k] = move(W.shard_tensor(full, v, rank, size, moe_mode))
        del raw
        out.update(W.build_layer(cfg, l, sh, rank, size, moe_mode))
        del sh
    return out


def write_checkpoint(cfg: ModelConfig, folder: str, seed: int = 0) -> None:
    """Writes config.json + one safetensors file per layer (CPU, real quantisation)."""
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    json.dump(cfg.to_hf_dict(), open(os.path.join(folder, "config.json"), "w"))
    e8 = quant.E8M0

    def fix(d):
        o = {}
        for k, v in d.items():
            if k.endswith(".scale") and v.dtype == torch.uint8 and e8 is not None:
                v = v.view(e8)
            o[k] = v.contiguous()
        return o

    save_file(fix(make_raw_top(cfg, "cpu", seed)), os.path.join(folder, "model-top.safetensors"))
    for l in range(cfg.num_layers):
        raw = {f"layers.{l}.{k}": v for k, v in make_raw_layer(cfg, l, "cpu", seed).items()}
        save_file(fix(raw), os.path.join(folder, f"model-layer{l:03d}.safetensors"))
