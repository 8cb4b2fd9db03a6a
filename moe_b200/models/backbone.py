"""Qwen3-style decoder with the two expert layouts.

Module and parameter names match the HuggingFace Qwen3-MoE tree that the reference subclasses
(`src/models/modeling_qwen3_moe.py:313-358,458-536,625-726`, `src/models/global_moe.py:45-151`),
so state dicts are interchangeable:
`model.embed_tokens`, `model.layers.N.{input_layernorm,post_attention_layernorm}`,
`model.layers.N.self_attn.{q,k,v,o}_proj / {q,k}_norm`, `model.layers.N.mlp.gate`,
`model.layers.N.mlp.experts.{gate_up_proj,down_proj}` (standard) or
`model.global_experts.{gate_up_proj,down_proj}` (global), `model.norm`, `lm_head`.

The forward keeps the residual stream and the normalised activations as a pair so that each
residual add is fused with the RMSNorm that follows it.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..utils.profiling import phase
from .config import Qwen3Config, Qwen3MoeConfig
from .router import DeepSeekRouter, TopKRouter, recompute_guard


class Linear(nn.Module):
    """Bias-free linear layer; `weight [out, in]`."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def forward(self, x):
        return ops.linear(x, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.variance_epsilon)


class Embedding(nn.Module):
    def __init__(self, num: int, dim: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num, dim))

    def forward(self, ids):
        return ops.embedding(ids, self.weight)


class Attention(nn.Module):
    """GQA attention with per-head QK RMSNorm before RoPE (`modeling_qwen3_moe.py:130-198`)."""

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.head_dim = config.head_dim
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.rope_theta = config.rope_theta
        self.eps = config.rms_norm_eps
        H = config.hidden_size
        self.q_proj = Linear(H, self.num_heads * self.head_dim)
        self.k_proj = Linear(H, self.num_kv_heads * self.head_dim)
        self.v_proj = Linear(H, self.num_kv_heads * self.head_dim)
        self.o_proj = Linear(self.num_heads * self.head_dim, H)
        self.q_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.k_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        # set by the training engine when q/k/v live side by side in the flat buffers:
        # (bf16 [N_qkv, H] view, fp32 gradient view)
        self._fused_qkv = None

    def forward(self, x):
        B, S, _ = x.shape
        q, k, v = ops.qkv_proj_norm_rope(x, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self._fused_qkv,
                                         self.q_norm.weight, self.k_norm.weight, B, S, self.num_heads,
                                         self.num_kv_heads, self.head_dim, self.rope_theta, self.eps)
        o = ops.attention(q, k, v)
        return self.o_proj(o.reshape(B, S, self.num_heads * self.head_dim))


class Experts(nn.Module):
    """Expert bank as two 3-D tensors (`modeling_qwen3_moe.py:217-254`)."""

    def __init__(self, config):
        super().__init__()
        self.num_experts = config.num_experts
        self.hidden_dim = config.hidden_size
        self.intermediate_dim = config.moe_intermediate_size
        ep_size = getattr(config, "ep_size", 1)
        self.num_local_experts = self.num_experts // ep_size
        self.gate_up_proj = nn.Parameter(torch.empty(self.num_local_experts, 2 * self.intermediate_dim, self.hidden_dim))
        self.down_proj = nn.Parameter(torch.empty(self.num_local_experts, self.hidden_dim, self.intermediate_dim))
        if ep_size > 1:  # this rank's slice of the bank along the expert dimension
            for p in (self.gate_up_proj, self.down_proj):
                p._ep_shard = (getattr(config, "ep_rank", 0), ep_size)

    def forward(self, hidden_states, top_k_index, top_k_weights):
        return ops.moe_experts(hidden_states, top_k_index, top_k_weights, self.gate_up_proj, self.down_proj)


class SparseMoeBlock(nn.Module):
    """Router + private expert bank (standard layout)."""

    def __init__(self, config, router_class=None):
        super().__init__()
        self.experts = Experts(config)
        self.gate = (router_class or TopKRouter)(config)

    def forward(self, x, global_experts=None):
        B, S, H = x.shape
        flat = x.reshape(-1, H)
        scores, w, idx = self.gate(flat)
        return self.experts(flat, idx, w).reshape(B, S, H), scores


class GlobalSparseMoeBlock(nn.Module):
    """Router only; the bank is owned by the model and passed in (`src/models/global_moe.py:45-66`)."""

    def __init__(self, config, router_class=None):
        super().__init__()
        self.gate = (router_class or TopKRouter)(config)

    def forward(self, x, global_experts):
        B, S, H = x.shape
        flat = x.reshape(-1, H)
        scores, w, idx = self.gate(flat)
        return global_experts(flat, idx, w).reshape(B, S, H), scores


class DenseMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate_proj = Linear(config.hidden_size, config.intermediate_size)
        self.up_proj = Linear(config.hidden_size, config.intermediate_size)
        self.down_proj = Linear(config.intermediate_size, config.hidden_size)
        self._fused_gate_up = None

    def forward(self, x, global_experts=None):
        return ops.swiglu_mlp(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight,
                              fused_gate_up=self._fused_gate_up), None


class DecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int, mlp: nn.Module):
        super().__init__()
        self.layer_idx = layer_idx
        self.self_attn = Attention(config, layer_idx)
        self.mlp = mlp
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, h, y, next_norm: RMSNorm, global_experts=None):
        """`h`: residual stream, `y = input_layernorm(h)`.  Returns (h', next_norm(h'), router scores)."""
        with phase("attn"):
            a = self.self_attn(y)
            h, y = ops.add_rmsnorm(a, h, self.post_attention_layernorm.weight,
                                   self.post_attention_layernorm.variance_epsilon)
        with phase("moe"):
            ops.set_moe_site(self.mlp, global_experts, self.layer_idx)
            m, scores = self.mlp(y, global_experts)
            h, y = ops.add_rmsnorm(m, h, next_norm.weight, next_norm.variance_epsilon)
        return h, y, scores


class DecoderModel(nn.Module):
    """Embedding, L decoder layers, final norm.  `layout`: 'standard' | 'global' | 'dense'."""

    def __init__(self, config, layout: str, router_class=None):
        super().__init__()
        self.config = config
        self.layout = layout
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size)
        if layout == "global":
            self.global_experts = Experts(config)
        layers = []
        for i in range(config.num_hidden_layers):
            if layout == "standard":
                mlp = SparseMoeBlock(config, router_class)
            elif layout == "global":
                mlp = GlobalSparseMoeBlock(config, router_class)
            else:
                mlp = DenseMLP(config)
            layers.append(DecoderLayer(config, i, mlp))
        self.layers = nn.ModuleList(layers)
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.gradient_checkpointing = False
        self._boundary_fn = None  # installed by the training engine (gradient-reduce overlap, parameter pulls)
        self._boundary_after_last = False  # engines that shard parameters also want a call in front of the head

    def forward(self, input_ids):
        """Returns (final normalised hidden states [B,S,H], tuple of per-layer router scores)."""
        h = self.embed_tokens(input_ids)
        first = self.layers[0].input_layernorm if len(self.layers) else self.norm
        y = ops.rmsnorm(h, first.weight, first.variance_epsilon)
        ge = self.global_experts if self.layout == "global" else None
        all_scores = []
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
            if self._boundary_fn is not None:
                h, y = self._boundary_fn(h, y, i)
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                h, y, scores = _checkpointed_layer(layer, h, y, nxt, ge)
            else:
                h, y, scores = layer(h, y, nxt, ge)
            if scores is not None:
                all_scores.append(scores)
        if self._boundary_fn is not None and self._boundary_after_last:
            h, y = self._boundary_fn(h, y, n)
        return y, tuple(all_scores)


class _LayerRunner:
    """Runs one layer; the second call (the recompute inside backward) is flagged so that
    routers do not count its tokens again."""

    def __init__(self, layer, nxt, ge):
        self.layer, self.nxt, self.ge, self.calls = layer, nxt, ge, 0

    def __call__(self, h, y):
        self.calls += 1
        if self.calls > 1:
            with recompute_guard():
                return self.layer(h, y, self.nxt, self.ge)
        return self.layer(h, y, self.nxt, self.ge)


def _checkpointed_layer(layer, h, y, nxt, ge):
    return checkpoint(_LayerRunner(layer, nxt, ge), h, y, use_reentrant=False)


def init_weights_(module: nn.Module, std: float = 0.02, generator: torch.Generator | None = None) -> None:
    """N(0, std) for every matrix / embedding / expert tensor / router, ones for norms
    (HF `_init_weights` as used by the reference models)."""
    for name, p in module.named_parameters():
        if name.endswith("norm.weight") or "layernorm" in name:
            with torch.no_grad():
                p.fill_(1.0)
        elif getattr(p, "_ep_shard", None) is not None:
            # draw the whole bank so that the values do not depend on the expert-parallel size, keep our slice
            r, n = p._ep_shard
            with torch.no_grad():
                full = torch.empty((p.shape[0] * n, *p.shape[1:]), dtype=p.dtype, device=p.device)
                full.normal_(mean=0.0, std=std, generator=generator)
                p.copy_(full[r * p.shape[0]:(r + 1) * p.shape[0]])
                del full
        else:
            with torch.no_grad():
                p.normal_(mean=0.0, std=std, generator=generator)
    for name, b in module.named_buffers():
        if name.endswith("expert_bias") or name.endswith("local_tokens_per_expert"):
            b.zero_()


__all__ = ["Linear", "RMSNorm", "Embedding", "Attention", "Experts", "SparseMoeBlock", "GlobalSparseMoeBlock",
           "DenseMLP", "DecoderLayer", "DecoderModel", "init_weights_", "TopKRouter", "DeepSeekRouter",
           "Qwen3Config", "Qwen3MoeConfig"]
