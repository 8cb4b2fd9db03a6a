"""Routing statistics (the reference's tests/test_routing_stats.py cases, including the
`utilization` and `expert_depth_coverage_*` keys that its code no longer emitted)."""
import math

import torch

from moe_b200.utils.routing_stats import accumulate_expert_counts, compute_routing_stats, expert_counts_to_tables


def uniform_probs(T=256, E=8, L=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(L):
        # every token prefers a different rotating pair of experts -> exactly uniform load
        p = torch.full((T, E), 0.01)
        for t in range(T):
            p[t, t % E] = 0.5
            p[t, (t + 1) % E] = 0.43
        out.append(p)
    return tuple(out)


def collapsed_probs(T=256, E=8, L=2):
    p = torch.full((T, E), 0.001)
    p[:, 0] = 0.6
    p[:, 1] = 0.393
    return tuple(p.clone() for _ in range(L))


def test_uniform_routing():
    s = compute_routing_stats(uniform_probs(), num_experts_per_tok=2)
    for l in (0, 1):
        tag = f"routing/layer_{l:02d}"
        assert abs(s[f"{tag}_load_imbalance"] - 1.0) < 1e-6
        assert s[f"{tag}_load_cv"] < 1e-6
        assert s[f"{tag}_num_active_experts"] == 8 and s[f"{tag}_utilization"] == 1.0
        assert abs(s[f"{tag}_entropy"] - 1.0) < 1e-4
        assert abs(s[f"{tag}_router_margin_mean"] - 0.42) < 1e-5
        assert len(s[f"_hist/{tag}_expert_load_frac"]) == 8
        assert abs(sum(s[f"_hist/{tag}_expert_load_frac"]) - 1.0) < 1e-6


def test_collapsed_routing():
    s = compute_routing_stats(collapsed_probs(), num_experts_per_tok=2)
    tag = "routing/layer_00"
    assert abs(s[f"{tag}_load_imbalance"] - 4.0) < 1e-6  # max / ideal = T / (2T/8)
    assert s[f"{tag}_num_active_experts"] == 2 and abs(s[f"{tag}_utilization"] - 0.25) < 1e-6
    assert s[f"{tag}_top_expert"] == 0
    assert abs(s[f"{tag}_entropy"] - math.log(2) / math.log(8)) < 1e-4
    assert s[f"{tag}_load_cv"] > 1.0
    assert isinstance(s[f"{tag}_num_active_experts"], int)


def test_global_cross_layer_metrics():
    same = compute_routing_stats(collapsed_probs(L=3), 2, is_global=True)
    assert abs(same["routing/cross_layer_sim_mean"] - 1.0) < 1e-5
    assert same["routing/global_pool_num_active"] == 2
    assert abs(same["routing/expert_depth_coverage_max"] - 1.0) < 1e-6
    assert abs(same["routing/expert_depth_coverage_mean"] - 0.25) < 1e-6
    assert same["_hist/global_expert_layer_count"][:3] == [3.0, 3.0, 0.0]
    a = torch.full((64, 8), 0.001); a[:, 0] = 0.6; a[:, 1] = 0.39
    b = torch.full((64, 8), 0.001); b[:, 4] = 0.6; b[:, 5] = 0.39
    disjoint = compute_routing_stats((a, b), 2, is_global=True)
    assert disjoint["routing/cross_layer_sim_mean"] < 1e-5
    assert disjoint["routing/global_pool_num_active"] == 4
    assert abs(disjoint["routing/global_pool_load_imbalance"] - 2.0) < 1e-5
    assert "routing/cross_layer_sim_mean" not in compute_routing_stats((a, b), 2, is_global=False)


def test_matches_direct_formulas_on_random_probs():
    torch.manual_seed(0)
    probs = (torch.softmax(torch.randn(300, 16) * 2, -1),)
    s = compute_routing_stats(probs, 4)
    _, idx = torch.topk(probs[0], 4, dim=-1)
    c = torch.bincount(idx.reshape(-1), minlength=16).float()
    assert abs(s["routing/layer_00_load_imbalance"] - (c.max() / (300 * 4 / 16)).item()) < 1e-5
    assert abs(s["routing/layer_00_load_cv"] - (c.std() / c.mean()).item()) < 1e-5
    sp, _ = probs[0].sort(-1, descending=True)
    assert abs(s["routing/layer_00_router_margin_min"] - (sp[:, 3] - sp[:, 4]).min().item()) < 1e-6


def test_accumulate_and_tables():
    probs = uniform_probs(T=64)
    acc = accumulate_expert_counts(probs, 2)
    acc = accumulate_expert_counts(probs, 2, acc)
    assert sorted(acc) == [0, 1] and torch.all(acc[0] == 32)
    sel = tuple(torch.zeros(64, 2, dtype=torch.long) for _ in probs)
    acc2 = accumulate_expert_counts(probs, 2, None, selected_experts=sel)
    assert acc2[0][0] == 128 and acc2[0][1:].sum() == 0
    t = expert_counts_to_tables(acc, is_global=True)
    assert t["_table/routing/layer_00_expert_tokens"][3] == (3, 32.0)
    assert t["_table/global_pool_expert_tokens"][0] == (0, 64.0)
