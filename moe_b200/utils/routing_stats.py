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
                          is_global: bool = False, counts: torch.Tensor | None = None,
                          margins: torch.Tensor | None = None, group=None, reduce_ranks: bool = False) -> dict:
    """`counts` (`[L, E]`) and `margins` (`[L, T]`, k-th minus (k+1)-th score per token) may come from the
    router kernels; otherwise both are taken from the recorded scores.  `reduce_ranks=True` sums the counts
    and margin statistics over the data-parallel ranks first (a collective: every rank must call), so the
    report describes the global batch and not only the calling rank's last micro-batch (the reference
    reports rank 0's, `train.py:638-643`)."""
    stats: dict = {}
    scalars: dict[str, torch.Tensor] = {}
    ints: set[str] = set()
    hists: dict[str, torch.Tensor] = {}
    loads = []
    K = num_experts_per_tok
    L = len(router_logits)
    if L == 0:
        return stats
    E = router_logits[0].shape[1]
    dev = router_logits[0].device
    if counts is None:
        counts = torch.stack([_counts_from_probs(p.detach().float(), K) for p in router_logits])
    counts = counts.float().clone()
    n_tok = torch.tensor([float(p.shape[0]) for p in router_logits], device=dev)
    have_margin = E > K
    if have_margin:
        if margins is None:
            tops = [topk_lowest_index(p.detach().float(), K + 1)[0] for p in router_logits]
            margins_l = [t[:, K - 1] - t[:, K] for t in tops]
            m_sum = torch.stack([m.sum() for m in margins_l])
            m_min = torch.stack([m.min() for m in margins_l])
        else:
            m_sum, m_min = margins.float().sum(dim=1), margins.float().min(dim=1).values
    if reduce_ranks and torch.distributed.is_available() and torch.distributed.is_initialized() \
            and torch.distributed.get_world_size(group) > 1:
        import torch.distributed as dist

        dist.all_reduce(counts, group=group)
        dist.all_reduce(n_tok, group=group)
        if have_margin:
            m_sum, m_min = m_sum.clone(), m_min.clone()
            dist.all_reduce(m_sum, group=group)
            dist.all_reduce(m_min, op=dist.ReduceOp.MIN, group=group)
    for li in range(L):
        tag = f"routing/layer_{li:02d}"
        c = counts[li]
        total = n_tok[li] * K
        ideal = total / E
        mean = c.mean()
        scalars[f"{tag}_load_imbalance"] = c.max() / ideal
        scalars[f"{tag}_load_cv"] = torch.where(mean > 0, c.std() / mean.clamp_min(1e-30), torch.zeros_like(mean))
        active = (c > 0).sum().float()
        scalars[f"{tag}_num_active_experts"] = active
        ints.add(f"{tag}_num_active_experts")
        scalars[f"{tag}_utilization"] = active / E
        scalars[f"{tag}_top_expert"] = c.argmax().float()
        ints.add(f"{tag}_top_expert")
        hists[f"_hist/{tag}_expert_load_frac"] = c / total
        ent = _entropy(c / (c.sum() + 1e-10))
        scalars[f"{tag}_entropy"] = ent / math.log(E) if E > 1 else torch.zeros_like(ent)
        if have_margin:
            scalars[f"{tag}_router_margin_mean"] = m_sum[li] / n_tok[li]
            scalars[f"{tag}_router_margin_min"] = m_min[li]
        loads.append(c)
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
