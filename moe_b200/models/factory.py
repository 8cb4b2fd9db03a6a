"""YAML -> model (`train.py:166-247` of the reference).

`model.type` is one of dense, standard_moe, deepseek_standard_moe, global_moe,
deepseek_global_moe.  Unknown keys are errors; keys the reference silently ignored
(`attention_bias`, `attention_dropout`, `output_router_logits`) are validated.
"""
from __future__ import annotations

import warnings

import torch
import yaml

from .causal_lm import (DeepSeekGlobalMoEForCausalLM, DeepSeekStandardMoEModel, GlobalMoEForCausalLM,
                        Qwen3ForCausalLM, StandardMoEModel)
from .config import GlobalMoEConfig, Qwen3Config, Qwen3MoeConfig

MODEL_TYPES = ("dense", "standard_moe", "deepseek_standard_moe", "global_moe", "deepseek_global_moe")

_COMMON_KEYS = {"type", "vocab_size", "hidden_size", "num_hidden_layers", "head_dim", "num_attention_heads",
                "num_key_value_heads", "intermediate_size", "max_position_embeddings", "rope_theta", "rms_norm_eps",
                "tie_word_embeddings", "attention_bias", "attention_dropout", "output_router_logits",
                "initializer_range"}
_MOE_KEYS = {"num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob", "router_aux_loss_coef",
             "seq_aux_loss_coef", "bias_update_rate", "bias_interpolation", "topk_scaling_factor", "num_groups",
             "group_topk", "experts_implementation", "score_fn", "expert_bias"}


def load_config(path: str) -> dict:
    with open(path) as f:
        return yaml.safe_load(f)


def model_config_from_dict(mcfg: dict, ep: tuple[int, int] | None = None):
    mtype = mcfg["type"]
    if mtype not in MODEL_TYPES:
        raise ValueError(f"Unknown model type: {mtype}")
    allowed = _COMMON_KEYS | (_MOE_KEYS if mtype != "dense" else set())
    unknown = set(mcfg) - allowed
    if unknown:
        raise ValueError(f"unknown model config keys for type {mtype}: {sorted(unknown)}")
    if mcfg.get("attention_bias", False):
        raise ValueError("attention_bias must be false")
    if mcfg.get("attention_dropout", 0.0) != 0.0:
        raise ValueError("attention_dropout must be 0.0")
    if mtype != "dense" and mcfg.get("output_router_logits", True) is not True:
        raise ValueError("output_router_logits must be true for MoE models")
    base = dict(
        vocab_size=mcfg["vocab_size"], hidden_size=mcfg["hidden_size"], num_hidden_layers=mcfg["num_hidden_layers"],
        head_dim=mcfg["head_dim"], num_attention_heads=mcfg["num_attention_heads"],
        num_key_value_heads=mcfg["num_key_value_heads"],
        max_position_embeddings=mcfg.get("max_position_embeddings", 32768),
        rope_theta=mcfg.get("rope_theta", 1_000_000.0), rms_norm_eps=mcfg.get("rms_norm_eps", 1e-6),
        tie_word_embeddings=mcfg.get("tie_word_embeddings", False),
        initializer_range=mcfg.get("initializer_range", 0.02),
    )
    if mtype == "dense":
        return Qwen3Config(intermediate_size=mcfg["intermediate_size"], **base)
    moe = dict(
        moe_intermediate_size=mcfg["moe_intermediate_size"],
        intermediate_size=mcfg.get("intermediate_size", mcfg["moe_intermediate_size"] * 4),
        router_aux_loss_coef=mcfg.get("router_aux_loss_coef", 0.001), norm_topk_prob=mcfg.get("norm_topk_prob", True),
        num_experts_per_tok=mcfg["num_experts_per_tok"], num_experts=mcfg["num_experts"], output_router_logits=True,
        score_fn=mcfg.get("score_fn"), expert_bias=mcfg.get("expert_bias"),
    )
    if mtype.startswith("deepseek") or mcfg.get("expert_bias") or mcfg.get("score_fn") == "sigmoid":
        moe.update(topk_scaling_factor=mcfg.get("topk_scaling_factor"), num_groups=mcfg.get("num_groups"),
                   group_topk=mcfg.get("group_topk"))
    if ep is not None and ep[1] > 1:
        moe.update(ep_rank=ep[0], ep_size=ep[1])
    cls = GlobalMoEConfig if "global" in mtype else Qwen3MoeConfig
    return cls(**base, **moe)


def build_model(cfg: dict, seed: int | None = None, device: str | torch.device | None = None,
                ep: tuple[int, int] | None = None):
    """Returns (model, model_config).  `cfg` is the whole YAML dict (uses `cfg['model']`).
    `ep=(rank, size)` shards every expert bank over `size` ranks (expert parallelism)."""
    mcfg = cfg["model"]
    config = model_config_from_dict(mcfg, ep)
    mtype = mcfg["type"]
    cls = {"dense": Qwen3ForCausalLM, "standard_moe": StandardMoEModel,
           "deepseek_standard_moe": DeepSeekStandardMoEModel, "global_moe": GlobalMoEForCausalLM,
           "deepseek_global_moe": DeepSeekGlobalMoEForCausalLM}[mtype]
    if device is not None:
        with torch.device(device):
            model = cls(config, seed=seed)
    else:
        model = cls(config, seed=seed)
    seq_coef = mcfg.get("seq_aux_loss_coef", 0.0) or 0.0
    if seq_coef > 0:
        model._seq_aux_loss_coef = seq_coef
    impl = mcfg.get("experts_implementation")
    if impl is not None:
        model.set_experts_implementation(impl)
    if mtype == "dense" and any(k in mcfg for k in ("num_experts", "num_experts_per_tok")):
        warnings.warn("MoE keys are ignored for a dense model")
    return model, config
