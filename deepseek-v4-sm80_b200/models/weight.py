"""Checkpoint loading: DeepSeek-V4 raw tensor names -> sharded runtime tensors.

The checkpoint format is the reference's, unchanged (python/minisgl/models/weight.py:19-215):
FP8 e4m3 dense weights with ``.scale`` e8m0 128x128 block scales, int8-packed FP4 experts with
e8m0 per-32 scales, FP32 state tensors, BF16 norms and embeddings; ``mtp.*`` is skipped.

Sharding rules (``tp`` ranks):
  * dim 0: ``attn.wq_b``, ``attn.wo_a``, ``attn.attn_sink``, shared experts ``w1``/``w3``, ``head`` (vocab rows)
  * dim 1: ``attn.wo_b``, shared experts ``w2``
  * routed experts: ``moe_mode="tp"`` splits w1/w3 on dim 0 and w2 on dim 1 (every rank holds every expert, the
    reference's layout); ``moe_mode="ep"`` keeps whole experts and gives rank r the experts
    ``[r*E/tp, (r+1)*E/tp)``.
  * everything else is replicated (``embed`` too: 1 GiB of HBM buys away one all-reduce per forward).
Merges: ``[wq_a; wkv] -> wqkv_a``, compressor ``[wkv; wgate] -> wkv_gate``, shared ``[w1; w3] -> gate_up``,
experts -> ``w13 [E, 2I, H/2]`` / ``w2 [E, H, I/2]``.  Block scales are decoded to fp32 once; ``wo_a`` (the one
projection the model applies to unquantised activations) is dequantised to bf16.

The loader works layer by layer so that at most one layer of raw tensors is alive next to the runtime copy.
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Callable, Dict, Iterable, List, Optional

import torch

from ..ops import quant
from .config import ModelConfig

SPLIT_DIM0 = ("attn.wq_b.", "attn.wo_a.", "attn.attn_sink", "ffn.shared_experts.w1.", "ffn.shared_experts.w3.")
SPLIT_DIM1 = ("attn.wo_b.", "ffn.shared_experts.w2.")
_EXPERT = re.compile(r"^layers\.(\d+)\.ffn\.experts\.(\d+)\.(w1|w2|w3)\.(weight|scale)$")


def remap_name(raw: str) -> str:
    """Raw checkpoint name -> the reference's runtime name (kept for parity with its state_dict keys)."""
    if raw == "embed.weight":
        return "model.embed_tokens.weight"
    if raw == "head.weight":
        return "lm_head.weight"
    if raw == "norm.weight":
        return "model.norm.weight"
    if raw.startswith("hc_head_"):
        return "model." + raw
    name = "model." + raw if raw.startswith("layers.") else raw
    name = name.replace(".attn.", ".self_attn.").replace(".ffn.", ".mlp.")
    name = name.replace(".attn_norm.", ".input_layernorm.").replace(".ffn_norm.", ".post_attention_layernorm.")
    if "self_attn" in name or "mlp" in name:
        name = name.replace(".scale", ".weight_scale_inv")
    name = name.replace(".gate.tid2eid", ".topk.tid2eid").replace(".gate.bias", ".gate.e_score_correction_bias")
    name = name.replace(".w1.", ".gate_proj.").replace(".w2.", ".down_proj.").replace(".w3.", ".up_proj.")
    return name


def shard_rows(n: int, rank: int, size: int):
    per = (n + size - 1) // size
    return rank * per, min((rank + 1) * per, n)


def shard_tensor(raw: str, t: torch.Tensor, rank: int, size: int, moe_mode: str = "tp") -> Optional[torch.Tensor]:
    """Returns this rank's shard of a raw tensor, or None when the rank does not own it (EP experts)."""
    if size == 1:
        return t
    if raw == "head.weight":
        a, b = shard_rows(t.shape[0], rank, size)
        return t[a:b].clone()
    m = _EXPERT.match(raw)
    if m is not None:
        if moe_mode == "ep":
            return t
        proj = m.group(3)
        return t.chunk(size, dim=0 if proj in ("w1", "w3") else 1)[rank].clone()
    for parts, dim in ((SPLIT_DIM0, 0), (SPLIT_DIM1, 1)):
        if any(p in raw for p in parts):
            if t.shape[dim] % size != 0:
                raise ValueError(f"{raw}: dim {dim} of shape {tuple(t.shape)} does not split over {size} ranks "
                                 "(block scales need shard sizes that are multiples of 128)")
            return t.chunk(size, dim=dim)[rank].clone()
    return t


def local_experts(cfg: ModelConfig, rank: int, size: int, moe_mode: str) -> range:
    if moe_mode == "ep" and size > 1:
        per = cfg.n_routed_experts // size
        return range(rank * per, (rank + 1) * per)
    return range(cfg.n_routed_experts)


def _scale_f32(t: torch.Tensor) -> torch.Tensor:
    return quant.e8m0_decode(t.view(torch.uint8) if t.dtype not in (torch.uint8, torch.float32) else t).contiguous()


def _u8(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def build_layer(cfg: ModelConfig, l: int, raw: Dict[str, torch.Tensor], rank: int, size: int,
                moe_mode: str = "tp") -> Dict[str, torch.Tensor]:
    """Turns the (already sharded) raw tensors of layer ``l`` (keys without the ``layers.l.`` prefix) into
    runtime tensors keyed ``L{l}.*``."""
    p = f"L{l}."
    out: Dict[str, torch.Tensor] = {}
    g = raw.__getitem__
    out[p + "attn_norm.weight"] = g("attn_norm.weight")
    out[p + "ffn_norm.weight"] = g("ffn_norm.weight")
    for k in ("hc_attn", "hc_ffn"):
        out[p + k + ".fn"] = g(k + "_fn").to(torch.bfloat16).contiguous()
        out[p + k + ".scale"] = g(k + "_scale").float().contiguous()
        out[p + k + ".base"] = g(k + "_base").float().contiguous()
    # attention
    out[p + "attn.wqkv_a.weight"] = torch.cat([g("attn.wq_a.weight"), g("attn.wkv.weight")], 0).contiguous()
    out[p + "attn.wqkv_a.scale"] = torch.cat([_scale_f32(g("attn.wq_a.scale")), _scale_f32(g("attn.wkv.scale"))], 0)
    for n in ("wq_b", "wo_b"):
        out[p + f"attn.{n}.weight"] = g(f"attn.{n}.weight").contiguous()
        out[p + f"attn.{n}.scale"] = _scale_f32(g(f"attn.{n}.scale"))
    out[p + "attn.wo_a.weight_bf16"] = quant.fp8_weight_dequant(
        g("attn.wo_a.weight"), _u8(g("attn.wo_a.scale")), dtype=torch.bfloat16).contiguous()
    out[p + "attn.q_norm.weight"] = g("attn.q_norm.weight")
    out[p + "attn.kv_norm.weight"] = g("attn.kv_norm.weight")
    out[p + "attn.sink"] = g("attn.attn_sink").float().contiguous()
    ratio = cfg.ratio(l)
    if ratio:
        out[p + "attn.comp.ape"] = g("attn.compressor.ape").float().contiguous()
        out[p + "attn.comp.wkv_gate"] = torch.cat(
            [g("attn.compressor.wkv.weight"), g("attn.compressor.wgate.weight")], 0).to(torch.bfloat16).contiguous()
        out[p + "attn.comp.norm"] = g("attn.compressor.norm.weight")
    if ratio == 4:
        out[p + "attn.idx.wq_b.weight"] = g("attn.indexer.wq_b.weight").contiguous()
        out[p + "attn.idx.wq_b.scale"] = _scale_f32(g("attn.indexer.wq_b.scale"))
        out[p + "attn.idx.weights_proj"] = g("attn.indexer.weights_proj.weight").to(torch.bfloat16).contiguous()
        out[p + "attn.idx.comp.ape"] = g("attn.indexer.compressor.ape").float().contiguous()
        idx_wkv_gate = torch.cat(
            [g("attn.indexer.compressor.wkv.weight"), g("attn.indexer.compressor.wgate.weight")], 0
        ).to(torch.bfloat16)
        # both compressors read the same activations: one stacked weight (one GEMM), the two parts are row views of it
        both = torch.cat([out[p + "attn.comp.wkv_gate"], idx_wkv_gate], 0).contiguous()
        n1 = out[p + "attn.comp.wkv_gate"].shape[0]
        out[p + "attn.comp_all.wkv_gate"] = both
        out[p + "attn.comp.wkv_gate"] = both[:n1]
        out[p + "attn.idx.comp.wkv_gate"] = both[n1:]
        out[p + "attn.idx.comp.norm"] = g("attn.indexer.compressor.norm.weight").float().contiguous()
    # MoE
    out[p + "moe.gate.weight"] = g("ffn.gate.weight").float().contiguous()
    out[p + "moe.gate.weight_bf16"] = g("ffn.gate.weight").to(torch.bfloat16).contiguous()  # tensor-core operand
    if "ffn.gate.tid2eid" in raw:
        out[p + "moe.gate.tid2eid"] = g("ffn.gate.tid2eid").to(torch.int32).contiguous()
    if "ffn.gate.bias" in raw:
        out[p + "moe.gate.bias"] = g("ffn.gate.bias").float().contiguous()
    experts = local_experts(cfg, rank, size, moe_mode)
    w13 = [torch.cat([g(f"ffn.experts.{e}.w1.weight"), g(f"ffn.experts.{e}.w3.weight")], 0) for e in experts]
    s13 = [torch.cat([_u8(g(f"ffn.experts.{e}.w1.scale")), _u8(g(f"ffn.experts.{e}.w3.scale"))], 0) for e in experts]
    for t in w13:
        if t.dtype != torch.int8:
            raise NotImplementedError(f"routed expert weights must be int8-packed fp4, got {t.dtype}")
    out[p + "moe.w13"] = torch.stack(w13, 0).contiguous()
    out[p + "moe.s13"] = torch.stack(s13, 0).contiguous()
    out[p + "moe.w2"] = torch.stack([g(f"ffn.experts.{e}.w2.weight") for e in experts], 0).contiguous()
    out[p + "moe.s2"] = torch.stack([_u8(g(f"ffn.experts.{e}.w2.scale")) for e in experts], 0).contiguous()
    from ..ops.cuda import MOE_KERNEL

    for key in ("moe.s13", "moe.s2"):
        sc = out[p + key]
        if MOE_KERNEL == "mx":
            # the block-scaled MMA takes every e8m0 byte as it is; 255 encodes NaN
            if sc.numel() and int(sc.max()) == 255:
                raise ValueError(f"{p + key}: expert scale byte 255 (NaN)")
            continue
        # the fp16 grouped GEMM applies a group scale as an fp16 power of two: exact for e8m0 bytes 103..142
        if sc.numel() and (int(sc.min()) < 103 or int(sc.max()) > 142):
            raise ValueError(f"{p + key}: expert scale bytes outside [103, 142] are not representable on the fp16 "
                             f"operand path (found {int(sc.min())}..{int(sc.max())})")
    out[p + "moe.sh_gate_up.weight"] = torch.cat(
        [g("ffn.shared_experts.w1.weight"), g("ffn.shared_experts.w3.weight")], 0).contiguous()
    out[p + "moe.sh_gate_up.scale"] = torch.cat(
        [_scale_f32(g("ffn.shared_experts.w1.scale")), _scale_f32(g("ffn.shared_experts.w3.scale"))], 0)
    out[p + "moe.sh_down.weight"] = g("ffn.shared_experts.w2.weight").contiguous()
    out[p + "moe.sh_down.scale"] = _scale_f32(g("ffn.shared_experts.w2.scale"))
    return out


def build_top(cfg: ModelConfig, raw: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {
        "embed.weight": raw["embed.weight"].to(torch.bfloat16),
        "head.weight": raw["head.weight"].to(torch.bfloat16).contiguous(),
        "norm.weight": raw["norm.weight"],
        "hc_head.fn": raw["hc_head_fn"].to(torch.bfloat16).contiguous(),
        "hc_head.scale": raw["hc_head_scale"].float().contiguous(),
        "hc_head.base": raw["hc_head_base"].float().contiguous(),
    }


def _index_checkpoint(folder: str) -> Dict[str, str]:
    idx = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(idx):
        wm = json.load(open(idx))["weight_map"]
        return {k: os.path.join(folder, v) for k, v in wm.items()}
    import safetensors

    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    files = [f for f in files if not f.endswith("consolidated.safetensors")] or files
    out = {}
    for f in files:
        with safetensors.safe_open(f, framework="pt", device="cpu") as h:
            for k in h.keys():
                out[k] = f
    return out


def load_checkpoint(folder: str, cfg: ModelConfig, device, rank: int = 0, size: int = 1, moe_mode: str = "tp",
                    progress: Optional[Callable[[str], None]] = None) -> Dict[str, torch.Tensor]:
    """Streams a DeepSeek-V4 safetensors checkpoint into sharded runtime tensors on ``device``."""
    import safetensors

    where = _index_checkpoint(folder)
    handles: Dict[str, object] = {}

    def fetch(name: str) -> torch.Tensor:
        f = where[name]
        if f not in handles:
            handles[f] = safetensors.safe_open(f, framework="pt", device=str(device))
        return handles[f].get_tensor(name)

    experts = set(local_experts(cfg, rank, size, moe_mode))
    weights: Dict[str, torch.Tensor] = {}
    top = {k: shard_tensor(k, fetch(k), rank, size, moe_mode)
           for k in ("embed.weight", "head.weight", "norm.weight", "hc_head_fn", "hc_head_scale", "hc_head_base")}
    weights.update(build_top(cfg, top))
    by_layer: Dict[int, List[str]] = {}
    for k in where:
        if k.startswith("layers."):
            li = int(k.split(".", 2)[1])
            if li < cfg.num_layers:
                by_layer.setdefault(li, []).append(k)
    for li in range(cfg.num_layers):
        raw = {}
        for k in by_layer.get(li, []):
            m = _EXPERT.match(k)
            if m is not None and int(m.group(2)) not in experts:
                continue
            raw[k.split(".", 2)[2]] = shard_tensor(k, fetch(k), rank, size, moe_mode)
        weights.update(build_layer(cfg, li, raw, rank, size, moe_mode))
        if progress:
            progress(f"layer {li}")
    return weights
