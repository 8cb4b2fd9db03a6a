"""Routers.

`TopKRouter` is the Qwen3-MoE softmax router (`src/models/modeling_qwen3_moe.py:257-275`);
`DeepSeekRouter` is the sigmoid router with a selection-only expert bias, optional
group-limited top-k, weight normalisation and a scaling factor
(`src/models/router.py:73-155`).  Score function and bias are orthogonal switches here, so a
softmax router can also carry the aux-loss-free bias.

Both return `(scores [T,E] fp32, weights [T,K], indices [T,K])`; `scores` is what the
reference records as `router_logits` (softmax probabilities or raw sigmoid scores).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..ops.oracle import group_limited_topk  # noqa: F401  (re-exported: reference API)

# Set while a checkpointed layer is being recomputed, so routers count each token once.
_RECOMPUTING = False


class recompute_guard:
    def __enter__(self):
        global _RECOMPUTING
        self.prev = _RECOMPUTING
        _RECOMPUTING = True

    def __exit__(self, *a):
        global _RECOMPUTING
        _RECOMPUTING = self.prev


class TopKRouter(nn.Module):
    score_fn = "softmax"
    use_bias = False

    def __init__(self, config, score_fn: str | None = None, expert_bias: bool | None = None):
        super().__init__()
        self.top_k = config.num_experts_per_tok
        self.num_experts = config.num_experts
        self.norm_topk_prob = config.norm_topk_prob
        self.hidden_dim = config.hidden_size
        self.score_fn = score_fn or getattr(config, "score_fn", None) or type(self).score_fn
        cfg_bias = getattr(config, "expert_bias", None)
        self.use_bias = type(self).use_bias if expert_bias is None and cfg_bias is None else bool(
            expert_bias if expert_bias is not None else cfg_bias)
        self.scaling_factor = getattr(config, "topk_scaling_factor", None) if self._uses_deepseek_extras() else None
        self.num_groups = getattr(config, "num_groups", None) if self._uses_deepseek_extras() else None
        self.group_topk = getattr(config, "group_topk", None) if self._uses_deepseek_extras() else None
        self.weight = nn.Parameter(torch.zeros(self.num_experts, self.hidden_dim))
        if self.use_bias:
            # persistent: part of the checkpoint; updated outside of autograd
            self.register_buffer("expert_bias", torch.zeros(self.num_experts, dtype=torch.float32))
        # per-step token counts, consumed and cleared by update_expert_biases
        self.register_buffer("local_tokens_per_expert", torch.zeros(self.num_experts, dtype=torch.float32),
                             persistent=False)
        self._last_top_k_idx = None
        # set by the model for one forward pass on the kernel path: where this router's statistics go
        self._site = None

    def separate_unbiased(self) -> bool:
        """Whether the unbiased top-k of the scores can differ from the selection."""
        return bool(self.use_bias or (self.num_groups or 0) > 1)

    def _uses_deepseek_extras(self) -> bool:
        return self.use_bias or self.score_fn == "sigmoid"

    def forward(self, hidden_states: torch.Tensor):
        x = hidden_states.reshape(-1, self.hidden_dim)
        bias = self.expert_bias if self.use_bias else None
        count = torch.is_grad_enabled() and not _RECOMPUTING
        site = self._site if ops.kernel_path(x) else None
        scores, weights, idx = ops.router(
            x, self.weight, bias, top_k=self.top_k, score_fn=self.score_fn, norm_topk_prob=self.norm_topk_prob,
            scaling_factor=self.scaling_factor, num_groups=self.num_groups, group_topk=self.group_topk, site=site,
            tokens_acc=self.local_tokens_per_expert if (site is not None and count) else None,
            collect=not _RECOMPUTING)
        self._last_top_k_idx = idx.detach()
        if count and site is None:
            with torch.no_grad():
                ones = torch.ones(idx.numel(), dtype=torch.float32, device=idx.device)
                self.local_tokens_per_expert.index_add_(0, idx.reshape(-1).long(), ones)
        if not hidden_states.is_cuda:
            weights = weights.to(hidden_states.dtype)
        return scores, weights, idx


class DeepSeekRouter(TopKRouter):
    """Sigmoid scores, bias-steered selection, unbiased weights (DeepSeek-V3 aux-loss-free balancing)."""

    score_fn = "sigmoid"
    use_bias = True
