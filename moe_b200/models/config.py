"""Model configuration objects.

Attribute names follow the HuggingFace Qwen3-MoE configuration so that code
written against the reference (`train.py:197-214`, `src/models/global_moe.py:34-42`)
reads the same fields here.  These are plain dataclasses: no hub, no JSON
round trip beyond `to_dict` / `from_dict`.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, fields
from typing import Any


@dataclass
class Qwen3Config:
    """Dense Qwen3 decoder (reference `train.py:176-194`)."""

    vocab_size: int = 151936
    hidden_size: int = 1024
    num_hidden_layers: int = 16
    head_dim: int = 128
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    intermediate_size: int = 3072
    max_position_embeddings: int = 32768
    rope_theta: float = 1_000_000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    attention_dropout: float = 0.0
    initializer_range: float = 0.02
    hidden_act: str = "silu"
    # MoE fields, zero for the dense model (the reference sets these dummies too)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    model_type: str = "qwen3"

    def __post_init__(self) -> None:
        if self.attention_bias:
            raise ValueError("attention_bias=True is not supported (every reference config sets false)")
        if self.attention_dropout != 0.0:
            raise ValueError("attention_dropout must be 0.0")
        if self.num_attention_heads % max(1, self.num_key_value_heads) != 0:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.hidden_act != "silu":
            raise ValueError("only SwiGLU (silu) experts are implemented")

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict[str, Any]):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})


@dataclass
class Qwen3MoeConfig(Qwen3Config):
    """Qwen3-MoE decoder: every layer is a sparse MoE layer.

    `num_experts` is the per-layer bank size for the standard layout.
    The DeepSeek-router extras (`topk_scaling_factor`, `num_groups`,
    `group_topk`) are ordinary fields here; the reference attaches them as
    ad-hoc attributes (`train.py:216-220`).
    """

    moe_intermediate_size: int = 768
    num_experts: int = 128
    num_experts_per_tok: int = 8
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.001
    output_router_logits: bool = True
    # router variants
    topk_scaling_factor: float | None = None
    num_groups: int | None = None
    group_topk: int | None = None
    # "softmax" | "sigmoid"; None = decided by the model class
    score_fn: str | None = None
    expert_bias: bool | None = None
    # expert parallelism: this process holds experts [ep_rank * E/ep_size, (ep_rank + 1) * E/ep_size)
    ep_size: int = 1
    ep_rank: int = 0
    model_type: str = "qwen3_moe"

    def __post_init__(self) -> None:
        super().__post_init__()
        if self.num_experts_per_tok > self.num_experts:
            raise ValueError("num_experts_per_tok cannot exceed num_experts")
        if (self.num_groups is None) != (self.group_topk is None):
            raise ValueError("num_groups and group_topk must be set together")
        if self.ep_size > 1 and self.num_experts % self.ep_size != 0:
            raise ValueError("num_experts must be divisible by ep_size")
        if self.num_groups is not None:
            if self.num_experts % self.num_groups != 0:
                raise ValueError("num_experts must be divisible by num_groups")
            if self.num_experts_per_tok % self.group_topk != 0:
                raise ValueError("num_experts_per_tok must be divisible by group_topk")


@dataclass
class GlobalMoEConfig(Qwen3MoeConfig):
    """`num_experts` is the size of the single bank shared by all layers."""

    num_experts: int = 2048
    model_type: str = "global_moe"


StandardMoEConfig = Qwen3MoeConfig
