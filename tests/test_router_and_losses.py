"""Router and load-balancing math on CPU, with the oracles inlined (Switch loss with one-hot masks,
DeepSeek-V3 Eq. 17-20 as written in the paper, Megatron-style group-limited top-k and bias update),
following the reference's tests/test_router_deepseek_v3.py, test_aux_loss_fix.py,
test_megatron_comparison.py and test_seq_loss_vs_paper.py."""
import math
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from moe_b200.models import DeepSeekRouter, TopKRouter, group_limited_topk
from moe_b200.models.load_balancing import load_balancing_loss_func, seq_load_balancing_loss_func


def cfg(**kw):
    d = dict(num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, hidden_size=64, topk_scaling_factor=None,
             num_groups=None, group_topk=None)
    d.update(kw)
    return SimpleNamespace(**d)


def make_router(cls=DeepSeekRouter, **kw):
    r = cls(cfg(**kw))
    torch.manual_seed(0)
    with torch.no_grad():
        r.weight.normal_(0, 0.5)
    return r


# ------------------------------------------------------------------ softmax router
def test_softmax_router_matches_hf_formula():
    r = make_router(TopKRouter, num_experts=16, num_experts_per_tok=4)
    x = torch.randn(32, 64)
    probs, w, idx = r(x)
    ref = torch.softmax(F.linear(x, r.weight), dim=-1, dtype=torch.float)
    tv, ti = torch.topk(ref, 4, dim=-1)
    assert torch.allclose(probs, ref, atol=1e-6)
    assert torch.equal(idx.sort(-1).values, ti.sort(-1).values)
    assert torch.allclose(w.sum(-1), torch.ones(32), atol=1e-5)
    assert torch.allclose(w, tv / tv.sum(-1, keepdim=True), atol=1e-6)
    assert not hasattr(r, "expert_bias")


def test_topk_ties_go_to_lowest_index():
    r = TopKRouter(cfg(num_experts=8, num_experts_per_tok=3))  # zero weights: exactly uniform probabilities
    _, _, idx = r(torch.randn(5, 64))
    assert torch.equal(idx, torch.tensor([[0, 1, 2]] * 5))


# ----------------------------------------------------------------- deepseek router
def test_fp32_gating_and_sigmoid_scores():
    r = make_router()
    x = torch.randn(16, 64)
    scores, w, idx = r(x)
    assert scores.dtype == torch.float32
    assert torch.allclose(scores, torch.sigmoid(F.linear(x.float(), r.weight.float())), atol=1e-6)
    assert (scores > 0).all() and (scores < 1).all()
    assert torch.allclose(w.sum(-1), torch.ones(16), atol=1e-5)


def test_bias_steers_selection_but_not_weights():
    r = make_router(num_experts=4, num_experts_per_tok=1, norm_topk_prob=False)
    x = torch.randn(64, 64)
    r.expert_bias.copy_(torch.tensor([0.0, 0.0, 0.0, 10.0]))
    scores, w, idx = r(x)
    assert (idx == 3).all()
    assert torch.allclose(w.squeeze(-1), scores[:, 3], atol=1e-6)  # weight = unbiased score


def test_eps_guard_and_scaling_factor():
    r = make_router(topk_scaling_factor=2.5)
    x = torch.randn(16, 64)
    _, w, _ = r(x)
    assert torch.allclose(w.sum(-1), torch.full((16,), 2.5), atol=1e-4)
    with torch.no_grad():
        r.weight.fill_(0)
        r.weight[:, 0] = -1000.0
    x = torch.zeros(4, 64)
    x[:, 0] = 1.0  # all scores ~ 0: the 1e-20 guard keeps the weights finite
    _, w, _ = r(x)
    assert torch.isfinite(w).all()


def _megatron_group_limited_topk(scores, topk, num_groups, group_topk):
    T, E = scores.shape
    gs = scores.view(T, num_groups, -1).topk(topk // group_topk, dim=-1)[0].sum(dim=-1)
    gi = torch.topk(gs, k=group_topk, dim=-1, sorted=False)[1]
    gm = torch.zeros_like(gs).scatter_(1, gi, 1)
    sm = gm.unsqueeze(-1).expand(T, num_groups, E // num_groups).reshape(T, -1)
    return torch.topk(scores.masked_fill(~sm.bool(), float("-inf")), k=topk, dim=-1)


def test_group_limited_topk_matches_megatron_and_respects_groups():
    torch.manual_seed(1)
    s = torch.rand(64, 32)
    v, i = group_limited_topk(s, 4, 8, 2)
    v2, i2 = _megatron_group_limited_topk(s, 4, 8, 2)
    assert torch.equal(i.sort(-1).values, i2.sort(-1).values) and torch.allclose(v.sort(-1).values, v2.sort(-1).values)
    assert ((i // 4).unique(dim=-1).shape[-1] <= 4)
    for row in (i // 4):
        assert len(set(row.tolist())) <= 2
    r = make_router(num_experts=32, num_experts_per_tok=4, num_groups=8, group_topk=2)
    _, _, idx = r(torch.randn(20, 64))
    for row in (idx // 4):
        assert len(set(row.tolist())) <= 2


def test_counts_accumulate_only_with_grad_enabled():
    r = make_router()
    x = torch.randn(16, 64)
    r(x)
    assert r.local_tokens_per_expert.sum().item() == 32
    r.local_tokens_per_expert.zero_()
    r.eval()
    with torch.no_grad():
        r(x)
    assert r.local_tokens_per_expert.sum() == 0
    assert r._last_top_k_idx.shape == (16, 2)
    sd = r.state_dict()
    assert "expert_bias" in sd and "local_tokens_per_expert" not in sd


def test_orthogonal_flags_softmax_with_bias():
    r = TopKRouter(cfg(num_experts=4, num_experts_per_tok=1), score_fn="softmax", expert_bias=True)
    assert hasattr(r, "expert_bias")
    r.expert_bias.copy_(torch.tensor([0.0, 5.0, 0.0, 0.0]))
    probs, w, idx = r(torch.randn(8, 64))
    assert (idx == 1).all() and torch.allclose(probs.sum(-1), torch.ones(8), atol=1e-5)


def test_gradients_flow_to_router_weight_through_weights():
    r = make_router()
    x = torch.randn(16, 64)
    _, w, _ = r(x)
    (w * torch.randn_like(w)).sum().backward()
    assert r.weight.grad is not None and r.weight.grad.abs().sum() > 0


# -------------------------------------------------------------------- switch loss
def _switch_oracle(gates, E, K):
    p = torch.cat(list(gates), 0)
    _, sel = torch.topk(p, K, dim=-1)
    mask = F.one_hot(sel, E).float()
    return (mask.mean(0) * p.mean(0).unsqueeze(0)).sum() * E


def test_switch_loss_uniform_is_topk_and_skew_is_larger():
    E, K, T = 128, 4, 512
    torch.manual_seed(0)
    noise = torch.rand(T, E) * 1e-6  # break ties uniformly
    uniform = (torch.full((T, E), 1.0 / E) + noise,)
    assert abs(load_balancing_loss_func(uniform, E, K).item() - K) < 0.05
    skew = torch.full((T, E), 1e-4)
    skew[:, :K] = (1 - 1e-4 * (E - K)) / K
    assert load_balancing_loss_func((skew,), E, K).item() > 10 * K


def test_switch_loss_matches_onehot_oracle_no_second_softmax():
    torch.manual_seed(0)
    gates = tuple(torch.softmax(torch.randn(64, 16) * 3, -1) for _ in range(3))
    ours = load_balancing_loss_func(gates, 16, 2)
    assert torch.allclose(ours, _switch_oracle(gates, 16, 2), atol=1e-5)
    double = _switch_oracle(tuple(torch.softmax(g, -1) for g in gates), 16, 2)
    assert abs(ours.item() - double.item()) > 1e-2
    assert load_balancing_loss_func(None) == 0 and load_balancing_loss_func(gates[0]) == 0


def test_switch_loss_gradient_is_through_probabilities_only():
    g = torch.softmax(torch.randn(32, 8), -1).requires_grad_()
    load_balancing_loss_func((g,), 8, 2).backward()
    _, sel = torch.topk(g.detach(), 2, dim=-1)
    cnt = torch.bincount(sel.reshape(-1), minlength=8).float()
    assert torch.allclose(g.grad, (8 * cnt / 32 ** 2).expand(32, 8), atol=1e-6)


def test_switch_loss_attention_mask():
    torch.manual_seed(0)
    B, S, E, K = 2, 8, 8, 2
    gates = tuple(torch.softmax(torch.randn(B * S, E), -1) for _ in range(2))
    mask = torch.ones(B, S)
    mask[1, 4:] = 0
    ours = load_balancing_loss_func(gates, E, K, attention_mask=mask)
    keep = mask.reshape(-1).bool()
    ref = _switch_oracle(tuple(g[keep] for g in gates), E, K)
    assert torch.allclose(ours, ref, atol=1e-5)


# ------------------------------------------------------------------ sequence loss
def _paper_seq_loss(scores, E, K, B):
    T = scores.shape[0]
    S = T // B
    sp = scores / scores.sum(-1, keepdim=True)
    total = 0.0
    for b in range(B):
        sb = sp[b * S:(b + 1) * S]
        _, sel = torch.topk(sb, K, dim=-1)
        f = torch.zeros(E)
        for t in range(S):
            for e in sel[t]:
                f[e] += 1
        f = f * E / (K * S)
        total = total + (f * sb.mean(0)).sum()
    return total / B


def test_seq_loss_matches_paper_and_uniform_is_one():
    torch.manual_seed(0)
    B, S, E, K = 3, 16, 8, 2
    layers = tuple(torch.sigmoid(torch.randn(B * S, E)) for _ in range(2))
    ours = seq_load_balancing_loss_func(layers, E, K, batch_size=B)
    ref = sum(_paper_seq_loss(l, E, K, B) for l in layers) / 2
    assert torch.allclose(ours, ref, atol=1e-5)
    uni = (torch.full((B * S, E), 0.3) + torch.rand(B * S, E) * 1e-6,)
    assert abs(seq_load_balancing_loss_func(uni, E, K, batch_size=B).item() - 1.0) < 0.05


def test_seq_loss_uses_actual_routing_when_given():
    torch.manual_seed(0)
    B, S, E, K = 2, 8, 8, 2
    s = (torch.sigmoid(torch.randn(B * S, E)),)
    forced = (torch.zeros(B * S, K, dtype=torch.long),)
    forced[0][:, 1] = 1
    a = seq_load_balancing_loss_func(s, E, K, batch_size=B, selected_experts=forced)
    sp = s[0] / s[0].sum(-1, keepdim=True)
    P = sp.reshape(B, S, E).mean(1)
    ref = ((E / K) * (P[:, 0] + P[:, 1])).mean()
    assert torch.allclose(a, ref, atol=1e-5)
    wrong_shape = (torch.zeros(3, K, dtype=torch.long),)
    b = seq_load_balancing_loss_func(s, E, K, batch_size=B, selected_experts=wrong_shape)
    assert torch.allclose(b, seq_load_balancing_loss_func(s, E, K, batch_size=B))
