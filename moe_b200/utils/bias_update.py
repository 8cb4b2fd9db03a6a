"""Aux-loss-free load balancing: per-step update of the routers' selection bias
(`train.py:67-139` of the reference; DeepSeek-V3 section 2.1.2).

`bias += sign(mean(counts) - counts) * rate`, with token counts summed over data-parallel ranks.
For the global layout the correction blends a per-layer term and a pooled (all layers) term:
`delta = alpha * delta_layer + (1 - alpha) * delta_global`, `alpha` decaying 1 -> 0 on a cosine.

All routers' counts travel in ONE `[L, E]` all-reduce (the reference issues L small ones) and the
bias statistics come back to the host in one transfer.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


def bias_alpha_schedule(step: int, warmup_steps: int = 5000) -> float:
    """Cosine decay 1 -> 0 over `warmup_steps`, then 0."""
    if step >= warmup_steps:
        return 0.0
    return 0.5 * (1 + math.cos(math.pi * step / max(1, warmup_steps)))


def _biased_routers(model) -> list:
    return [m for m in model.modules() if getattr(m, "use_bias", False) and hasattr(m, "expert_bias")]


def _num_processes(accelerator) -> int:
    if accelerator is not None and hasattr(accelerator, "num_processes"):
        return int(accelerator.num_processes)
    return dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1


@torch.no_grad()
def update_expert_biases(model, update_rate: float, accelerator=None, is_global: bool = False, alpha: float = 0.0,
                         group=None) -> dict:
    """Returns `routing/expert_bias_{mean,std,min,max}` (empty dict when no router carries a bias).

    `accelerator` is anything with `.num_processes` (kept for call compatibility) or None, in which
    case the default process group decides."""
    routers = _biased_routers(model)
    if not routers:
        return {}
    same = len({r.num_experts for r in routers}) == 1
    if same:
        counts = torch.stack([r.local_tokens_per_expert for r in routers])  # [L, E]
        if _num_processes(accelerator) > 1 and dist.is_initialized():
            dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=group)
        per_router = list(counts.unbind(0))
    else:
        per_router = []
        for r in routers:
            c = r.local_tokens_per_expert.clone()
            if _num_processes(accelerator) > 1 and dist.is_initialized():
                dist.all_reduce(c, op=dist.ReduceOp.SUM, group=group)
            per_router.append(c)
    for r in routers:
        r.local_tokens_per_expert.zero_()
    if is_global:
        gcounts = torch.stack(per_router).sum(0)
        gdelta = torch.sign(gcounts.mean() - gcounts) * update_rate
        for r, c in zip(routers, per_router):
            if alpha > 0:
                ldelta = torch.sign(c.mean() - c) * update_rate
                r.expert_bias += alpha * ldelta + (1 - alpha) * gdelta
            else:
                r.expert_bias += gdelta
    else:
        for r, c in zip(routers, per_router):
            r.expert_bias += torch.sign(c.mean() - c) * update_rate
    allb = torch.cat([r.expert_bias for r in routers])
    vals = torch.stack([allb.mean(), allb.std(), allb.min(), allb.max()]).cpu().tolist()
    return dict(zip(["routing/expert_bias_mean", "routing/expert_bias_std", "routing/expert_bias_min",
                     "routing/expert_bias_max"], vals))


def get_selected_experts_for_seq_aux(model):
    """Last routed (biased) top-k indices of every layer's router, or None if any is missing."""
    layers = getattr(getattr(model, "model", None), "layers", None)
    if layers is None:
        return None
    sel = []
    for layer in layers:
        gate = getattr(getattr(layer, "mlp", None), "gate", None)
        idx = getattr(gate, "_last_top_k_idx", None)
        if idx is None:
            return None
        sel.append(idx)
    return tuple(sel) if sel else None
