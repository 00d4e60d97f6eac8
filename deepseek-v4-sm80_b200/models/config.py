"""Model hyper-parameters of the DeepSeek-V4 family.

``ModelConfig.from_hf`` accepts a HuggingFace ``config.json`` (dict or PretrainedConfig)
and rejects everything that is not ``DeepseekV4ForCausalLM`` / ``deepseek_v4``, like the
reference (python/minisgl/models/config.py:81-204).  ``flash()`` holds the full
DeepSeek-V4-Flash shape, ``tiny()`` the CPU test model; ``with_layers`` derives
depth-reduced variants with unchanged per-layer shapes.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, List, Optional


@dataclass(frozen=True)
class ModelConfig:
    num_layers: int = 43
    hidden_size: int = 4096
    num_heads: int = 64
    head_dim: int = 512
    rope_head_dim: int = 64
    q_lora_rank: int = 1024
    o_lora_rank: int = 1024
    o_groups: int = 8
    window_size: int = 128
    compress_ratios: tuple = ()
    index_topk: int = 512
    index_head_dim: int = 128
    index_n_heads: int = 64
    n_routed_experts: int = 256
    num_experts_per_tok: int = 6
    n_shared_experts: int = 1
    moe_intermediate_size: int = 2048
    scoring_func: str = "sqrtsoftplus"
    routed_scaling_factor: float = 1.5
    swiglu_limit: Optional[float] = 7.0
    n_hash_layers: int = 3
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    vocab_size: int = 129280
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    compress_rope_theta: Optional[float] = 160000.0
    original_seq_len: int = 65536
    rope_factor: float = 16.0
    beta_fast: int = 32
    beta_slow: int = 1
    max_position: int = 1048576
    expert_dtype: str = "fp4"
    model_type: str = "deepseek_v4"
    architectures: tuple = ("DeepseekV4ForCausalLM",)
    bos_token_id: int = 0
    eos_token_id: int = 1

    # ------------------------------------------------------------------ derived
    @property
    def nope_head_dim(self) -> int:
        return self.head_dim - self.rope_head_dim

    def ratio(self, layer: int) -> int:
        return self.compress_ratios[layer] if layer < len(self.compress_ratios) else 0

    @property
    def c4_layers(self) -> List[int]:
        return [i for i in range(self.num_layers) if self.ratio(i) == 4]

    @property
    def c128_layers(self) -> List[int]:
        return [i for i in range(self.num_layers) if self.ratio(i) == 128]

    def with_layers(self, n: int) -> "ModelConfig":
        """Depth-reduced variant: the first n layers' ratio pattern, every per-layer shape unchanged."""
        ratios = tuple(self.compress_ratios[:n])
        return dataclasses.replace(self, num_layers=n, compress_ratios=ratios,
                                   n_hash_layers=min(self.n_hash_layers, n))

    # ------------------------------------------------------------------ presets
    @staticmethod
    def flash() -> "ModelConfig":
        # layers 0,1 dense-window only; then alternating ratio 4 / 128 (compress_ratios[2:4] == [4, 128])
        ratios = tuple([0, 0] + [4 if (i % 2 == 0) else 128 for i in range(41)])
        return ModelConfig(compress_ratios=ratios)

    @staticmethod
    def tiny(**over) -> "ModelConfig":
        """2 layers, hidden 256, 4 heads of 64, vocab 1024, indexer 2x32 top-64, ratios (4, 128), window 128,
        8 routed experts top-2 (inter 512) + 1 shared."""
        base = dict(
            num_layers=2, hidden_size=256, num_heads=4, head_dim=64, rope_head_dim=16, q_lora_rank=128,
            o_lora_rank=128, o_groups=2, window_size=128, compress_ratios=(4, 128), index_topk=64,
            index_head_dim=32, index_n_heads=2, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
            moe_intermediate_size=512, n_hash_layers=0, vocab_size=1024, original_seq_len=0, rope_factor=1.0,
            max_position=8192, compress_rope_theta=40000.0,
        )
        base.update(over)
        return ModelConfig(**base)

    # ------------------------------------------------------------------ HF
    @staticmethod
    def from_hf(cfg: Any) -> "ModelConfig":
        get = (lambda k, d=None: cfg.get(k, d)) if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
        arch = get("architectures")
        if not arch or list(arch)[0] != "DeepseekV4ForCausalLM":
            raise ValueError(f"Model architecture {arch!r} is not supported; this engine serves DeepSeek V4 only "
                             "(DeepseekV4ForCausalLM).")
        if get("model_type") != "deepseek_v4":
            raise ValueError(f"Model type {get('model_type')!r} is not supported (expected 'deepseek_v4').")
        n_layers = get("num_hidden_layers")
        rs = get("rope_scaling") or {}
        head_dim = get("head_dim") or get("hidden_size") // get("num_attention_heads")
        ratios = tuple(get("compress_ratios") or [0] * n_layers)
        eos = get("eos_token_id", 1)
        if isinstance(eos, (list, tuple)):
            eos = eos[0]
        return ModelConfig(
            num_layers=n_layers, hidden_size=get("hidden_size"), num_heads=get("num_attention_heads"),
            head_dim=head_dim, rope_head_dim=get("qk_rope_head_dim", head_dim), q_lora_rank=get("q_lora_rank", 0) or 0,
            o_lora_rank=get("o_lora_rank", 0) or 0, o_groups=get("o_groups", 1) or 1,
            window_size=get("window_size", get("sliding_window", 0)), compress_ratios=ratios,
            index_topk=get("index_topk", 0) or 0, index_head_dim=get("index_head_dim", 0) or 0,
            index_n_heads=get("index_n_heads", 0) or 0, n_routed_experts=get("n_routed_experts", 0),
            num_experts_per_tok=get("num_experts_per_tok", 0), n_shared_experts=get("n_shared_experts", 0) or 0,
            moe_intermediate_size=get("moe_intermediate_size", 0), scoring_func=get("scoring_func", ""),
            routed_scaling_factor=get("routed_scaling_factor", 1.0), swiglu_limit=get("swiglu_limit"),
            n_hash_layers=get("num_hash_layers", get("n_hash_layers", 0)) or 0, hc_mult=get("hc_mult", 1) or 1,
            hc_sinkhorn_iters=get("hc_sinkhorn_iters", 0) or 0, hc_eps=get("hc_eps", 1e-6),
            vocab_size=get("vocab_size"), rms_norm_eps=get("rms_norm_eps", 1e-6),
            rope_theta=get("rope_theta") or rs.get("rope_theta") or 10000.0,
            compress_rope_theta=get("compress_rope_theta"),
            original_seq_len=int(rs.get("original_max_position_embeddings", 0) or 0),
            rope_factor=float(rs.get("factor", 1.0) or 1.0), beta_fast=int(rs.get("beta_fast", 32) or 32),
            beta_slow=int(rs.get("beta_slow", 1) or 1), max_position=get("max_position_embeddings", 1048576),
            expert_dtype=get("expert_dtype", "fp4"), bos_token_id=get("bos_token_id", 0) or 0, eos_token_id=eos,
        )

    def to_hf_dict(self) -> dict:
        """The inverse of from_hf, used when writing synthetic checkpoints."""
        return {
            "architectures": list(self.architectures), "model_type": self.model_type,
            "num_hidden_layers": self.num_layers, "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_heads, "num_key_value_heads": 1, "head_dim": self.head_dim,
            "qk_rope_head_dim": self.rope_head_dim, "qk_nope_head_dim": self.nope_head_dim,
            "q_lora_rank": self.q_lora_rank, "o_lora_rank": self.o_lora_rank, "o_groups": self.o_groups,
            "window_size": self.window_size, "compress_ratios": list(self.compress_ratios),
            "index_topk": self.index_topk, "index_head_dim": self.index_head_dim,
            "index_n_heads": self.index_n_heads, "n_routed_experts": self.n_routed_experts,
            "num_experts_per_tok": self.num_experts_per_tok, "n_shared_experts": self.n_shared_experts,
            "moe_intermediate_size": self.moe_intermediate_size, "scoring_func": self.scoring_func,
            "routed_scaling_factor": self.routed_scaling_factor, "swiglu_limit": self.swiglu_limit,
            "num_hash_layers": self.n_hash_layers, "hc_mult": self.hc_mult,
            "hc_sinkhorn_iters": self.hc_sinkhorn_iters, "hc_eps": self.hc_eps, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "compress_rope_theta": self.compress_rope_theta,
            "rope_scaling": {"original_max_position_embeddings": self.original_seq_len, "factor": self.rope_factor,
                             "beta_fast": self.beta_fast, "beta_slow": self.beta_slow},
            "max_position_embeddings": self.max_position, "expert_dtype": self.expert_dtype,
            "hidden_act": "silu", "bos_token_id": self.bos_token_id, "eos_token_id": self.eos_token_id,
        }
