"""Routing statistics from the recorded per-layer router scores.

Same keys as the reference (`src/utils/routing_stats.py:53-220`): per layer
`routing/layer_NN_{load_imbalance, load_cv, num_active_experts, top_expert, entropy,
router_margin_mean, router_margin_min}` and `_hist/routing/layer_NN_expert_load_frac`; for the
global layout `routing/cross_layer_sim_{mean,min,max}`, `routing/global_pool_*` and the two
`_hist/global_*` lists.  Added here: `routing/layer_NN_utilization` (fraction of experts that got
a token) and `routing/expert_depth_coverage_{mean,max}` (share of layers that use an expert).

Everything is computed on the device that holds the scores and brought to the host in one
transfer at the end (the reference synchronises once per scalar).  Top-k ties go to the lowest
expert index.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from ..ops.oracle import topk_lowest_index


def _counts_from_probs(probs: torch.Tensor, k: int) -> torch.Tensor:
    _, idx = topk_lowest_index(probs, k)
    E = probs.shape[1]
    flat = idx.reshape(-1)
    return torch.zeros(E, dtype=torch.float32, device=probs.device).index_add_(
        0, flat, torch.ones(flat.numel(), dtype=torch.float32, device=probs.device))


def accumulate_expert_counts(router_logits: Sequence[torch.Tensor], num_experts_per_tok: int,
                             accumulator: dict[int, torch.Tensor] | None = None,
                             selected_experts: Sequence[torch.Tensor] | None = None) -> dict[int, torch.Tensor]:
    """Add this batch's per-layer expert token counts into `{layer: [E] counts}`.

    `selected_experts` (the routers' own choices) skips the top-k; without it counts come from the
    top-k of the scores, as in the reference."""
    if accumulator is None:
        accumulator = {}
    for li, probs in enumerate(router_logits):
        if selected_experts is not None and selected_experts[li] is not None:
            idx = selected_experts[li].reshape(-1).long()
            E = probs.shape[1]
            counts = torch.zeros(E, dtype=torch.float32, device=idx.device).index_add_(
                0, idx, torch.ones(idx.numel(), dtype=torch.float32, device=idx.device))
        else:
            counts = _counts_from_probs(probs.detach().float(), num_experts_per_tok)
        if li in accumulator:
            accumulator[li] += counts
        else:
            accumulator[li] = counts
    return accumulator


def expert_counts_to_tables(accumulator: dict[int, torch.Tensor], is_global: bool = False) -> dict:
    """`_table/routing/layer_NN_expert_tokens` lists of (expert, count); plus the pooled table for global."""
    stats = {}
    for li in sorted(accumulator):
        c = accumulator[li].cpu().tolist()
        stats[f"_table/routing/layer_{li:02d}_expert_tokens"] = list(zip(range(len(c)), c))
    if is_global and len(accumulator) > 1:
        pool = torch.stack([accumulator[i] for i in sorted(accumulator)]).sum(0).cpu().tolist()
        stats["_table/global_pool_expert_tokens"] = list(zip(range(len(pool)), pool))
    return stats


def _entropy(dist_: torch.Tensor) -> torch.Tensor:
    return -(dist_ * (dist_ + 1e-10).log()).sum()


def compute_routing_stats(router_logits: Sequence[torch.Tensor], num_experts_per_tok: int,
                          is_global: bool = False) -> dict:
    stats: dict = {}
    scalars: dict[str, torch.Tensor] = {}
    ints: set[str] = set()
    hists: dict[str, torch.Tensor] = {}
    loads = []
    K = num_experts_per_tok
    for li, probs in enumerate(router_logits):
        probs = probs.detach().float()
        T, E = probs.shape
        tag = f"routing/layer_{li:02d}"
        counts = _counts_from_probs(probs, K)
        total = float(T * K)
        ideal = total / E
        mean = counts.mean()
        scalars[f"{tag}_load_imbalance"] = counts.max() / ideal
        scalars[f"{tag}_load_cv"] = torch.where(mean > 0, counts.std() / mean.clamp_min(1e-30), torch.zeros_like(mean))
        active = (counts > 0).sum().float()
        scalars[f"{tag}_num_active_experts"] = active
        ints.add(f"{tag}_num_active_experts")
        scalars[f"{tag}_utilization"] = active / E
        scalars[f"{tag}_top_expert"] = counts.argmax().float()
        ints.add(f"{tag}_top_expert")
        hists[f"_hist/{tag}_expert_load_frac"] = counts / total
        ent = _entropy(counts / (counts.sum() + 1e-10))
        scalars[f"{tag}_entropy"] = ent / math.log(E) if E > 1 else torch.zeros_like(ent)
        if E > K:
            top = topk_lowest_index(probs, K + 1)[0]
            margin = top[:, K - 1] - top[:, K]
            scalars[f"{tag}_router_margin_mean"] = margin.mean()
            scalars[f"{tag}_router_margin_min"] = margin.min()
        loads.append(counts)
    if is_global and len(loads) > 1:
        mat = torch.stack(loads).float()
        L, E = mat.shape
        normed = mat / mat.norm(dim=1, keepdim=True).clamp(min=1e-10)
        sim = normed @ normed.T
        off = sim[torch.triu(torch.ones(L, L, dtype=torch.bool, device=mat.device), diagonal=1)]
        scalars["routing/cross_layer_sim_mean"] = off.mean()
        scalars["routing/cross_layer_sim_min"] = off.min()
        scalars["routing/cross_layer_sim_max"] = off.max()
        layer_count = (mat > 0).float().sum(0)
        hists["_hist/global_expert_layer_count"] = layer_count
        scalars["routing/expert_depth_coverage_mean"] = (layer_count / L).mean()
        scalars["routing/expert_depth_coverage_max"] = (layer_count / L).max()
        pool = mat.sum(0)
        pool_total = pool.sum()
        pmean = pool.mean()
        scalars["routing/global_pool_load_imbalance"] = pool.max() / (pool_total / E)
        scalars["routing/global_pool_load_cv"] = torch.where(pmean > 0, pool.std() / pmean.clamp_min(1e-30),
                                                             torch.zeros_like(pmean))
        scalars["routing/global_pool_num_active"] = (pool > 0).sum().float()
        ints.add("routing/global_pool_num_active")
        scalars["routing/global_pool_top_expert"] = pool.argmax().float()
        ints.add("routing/global_pool_top_expert")
        frac = pool / pool_total
        hists["_hist/global_pool_expert_load_frac"] = frac
        pe = _entropy(frac)
        scalars["routing/global_pool_entropy"] = pe / math.log(E) if E > 1 else torch.zeros_like(pe)
    if scalars:
        keys = list(scalars)
        vals = torch.stack([scalars[k].reshape(()).float() for k in keys]).cpu().tolist()  # one transfer
        for k, v in zip(keys, vals):
            stats[k] = int(round(v)) if k in ints else v
    for k, h in hists.items():
        stats[k] = h.cpu().tolist()
    return stats
