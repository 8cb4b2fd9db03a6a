"""Model classes (same public names as the reference's `src/models/__init__.py:1-26`)."""
from .backbone import (Attention, DecoderLayer, DecoderModel, DenseMLP, Embedding, Experts, GlobalSparseMoeBlock,
                       Linear, RMSNorm, SparseMoeBlock, init_weights_)
from .causal_lm import (DeepSeekGlobalMoEForCausalLM, DeepSeekStandardMoEModel, GlobalMoEForCausalLM, GlobalMoEModel,
                        MoeCausalLMOutput, Qwen3ForCausalLM, Qwen3MoeForCausalLM, StandardMoEModel)
from .config import GlobalMoEConfig, Qwen3Config, Qwen3MoeConfig, StandardMoEConfig
from .factory import build_model, load_config
from .load_balancing import load_balancing_loss_func, seq_load_balancing_loss_func
from .router import DeepSeekRouter, TopKRouter, group_limited_topk

__all__ = [
    "Qwen3MoeConfig", "Qwen3MoeForCausalLM", "Qwen3Config", "Qwen3ForCausalLM", "StandardMoEConfig",
    "StandardMoEModel", "DeepSeekStandardMoEModel", "DeepSeekRouter", "TopKRouter", "GlobalMoEConfig",
    "GlobalMoEModel", "GlobalMoEForCausalLM", "DeepSeekGlobalMoEForCausalLM", "group_limited_topk",
    "load_balancing_loss_func", "seq_load_balancing_loss_func", "build_model", "load_config", "MoeCausalLMOutput",
]
