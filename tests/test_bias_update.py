"""Aux-loss-free bias update (reference tests/test_router_deepseek_v3.py:331-666, test_megatron_comparison.py)."""
import math
from types import SimpleNamespace

import torch
import torch.nn as nn

from helpers import batch, tiny_cfg
from moe_b200.models import DeepSeekRouter, build_model
from moe_b200.utils.bias_update import bias_alpha_schedule, get_selected_experts_for_seq_aux, update_expert_biases


def routers(n=3, E=4):
    cfg = SimpleNamespace(num_experts=E, num_experts_per_tok=1, norm_topk_prob=True, hidden_size=8,
                          topk_scaling_factor=None, num_groups=None, group_topk=None)
    return nn.ModuleList([DeepSeekRouter(cfg) for _ in range(n)])


def megatron_updated_bias(tokens_per_expert, bias, rate):
    avg = tokens_per_expert.sum(dim=-1, keepdim=True) / tokens_per_expert.shape[-1]
    return bias + torch.sign(avg - tokens_per_expert) * rate


def test_standard_update_matches_megatron_and_clears_counts():
    m = routers()
    counts = [torch.tensor([10.0, 0, 5, 5]), torch.tensor([1.0, 1, 1, 1]), torch.tensor([0.0, 9, 0, 3])]
    for r, c in zip(m, counts):
        r.local_tokens_per_expert.copy_(c)
    stats = update_expert_biases(m, 1e-3, SimpleNamespace(num_processes=1))
    for r, c in zip(m, counts):
        assert torch.allclose(r.expert_bias, megatron_updated_bias(c, torch.zeros(4), 1e-3))
        assert r.local_tokens_per_expert.sum() == 0
    allb = torch.cat([r.expert_bias for r in m])
    assert abs(stats["routing/expert_bias_mean"] - allb.mean().item()) < 1e-9
    assert abs(stats["routing/expert_bias_std"] - allb.std().item()) < 1e-9
    assert set(stats) == {"routing/expert_bias_mean", "routing/expert_bias_std", "routing/expert_bias_min",
                          "routing/expert_bias_max"}


def test_global_update_pools_layers_and_interpolates():
    counts = [torch.tensor([10.0, 0, 0, 0]), torch.tensor([0.0, 0, 6, 0])]
    pooled = torch.stack(counts).sum(0)
    gdelta = torch.sign(pooled.mean() - pooled) * 1e-3
    m = routers(2)
    for r, c in zip(m, counts):
        r.local_tokens_per_expert.copy_(c)
    update_expert_biases(m, 1e-3, None, is_global=True, alpha=0.0)
    for r in m:
        assert torch.allclose(r.expert_bias, gdelta)
    m = routers(2)
    for r, c in zip(m, counts):
        r.local_tokens_per_expert.copy_(c)
    update_expert_biases(m, 1e-3, None, is_global=True, alpha=0.25)
    for r, c in zip(m, counts):
        ld = torch.sign(c.mean() - c) * 1e-3
        assert torch.allclose(r.expert_bias, 0.25 * ld + 0.75 * gdelta)


def test_no_biased_routers_is_a_no_op():
    model, _ = build_model(tiny_cfg("standard_moe"))
    assert update_expert_biases(model, 1e-3, None) == {}


def test_alpha_schedule():
    assert bias_alpha_schedule(0) == 1.0
    assert abs(bias_alpha_schedule(2500) - 0.5) < 1e-9
    assert bias_alpha_schedule(5000) == 0.0 and bias_alpha_schedule(10 ** 6) == 0.0
    vals = [bias_alpha_schedule(s) for s in range(0, 5001, 250)]
    assert all(a >= b for a, b in zip(vals, vals[1:]))
    assert abs(bias_alpha_schedule(100, warmup_steps=200) - 0.5) < 1e-9


def test_real_model_loop_balances_load():
    torch.manual_seed(0)
    model, _ = build_model(tiny_cfg("deepseek_standard_moe", num_groups=None, group_topk=None), seed=0)
    with torch.no_grad():  # a router that strongly prefers expert 0
        for r in model.routers():
            r.weight.zero_()
            r.expert_bias.zero_()
            r.expert_bias[0] = 0.02
    ids = batch(B=4, S=32)
    first = None
    seen = torch.zeros(8)
    for step in range(40):
        model(input_ids=ids, labels=ids, output_router_logits=True)
        sel = get_selected_experts_for_seq_aux(model)
        assert sel is not None and sel[0].shape == (128, 2)
        c = model.routers()[0].local_tokens_per_expert.clone()
        first = c if first is None else first
        seen += (c > 0).float()
        update_expert_biases(model, 1e-3, None)
    assert first[0] == 128 and (first > 0).sum() == 2  # everyone picked experts 0 and 1 at first
    assert (seen > 0).all()  # the bias walk brought every expert into use
