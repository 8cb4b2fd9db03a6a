"""Model wiring on CPU (the reference's tests/test_models.py, test_integration.py and
test_ce_loss_diagnosis.py cases, against this package's classes)."""
import glob
import math
import os

import pytest
import torch

from helpers import batch, tiny_cfg
from moe_b200.models import (DeepSeekGlobalMoEForCausalLM, DeepSeekRouter, DeepSeekStandardMoEModel,
                             GlobalMoEForCausalLM, StandardMoEModel, build_model, load_config)
from moe_b200.models.factory import model_config_from_dict
from moe_b200.models.load_balancing import load_balancing_loss_func, seq_load_balancing_loss_func

MOE_TYPES = ["standard_moe", "deepseek_standard_moe", "global_moe", "deepseek_global_moe"]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_yaml_config_parses():
    files = sorted(glob.glob(os.path.join(ROOT, "configs", "**", "*.yaml"), recursive=True))
    assert len(files) >= 25
    for f in files:
        cfg = load_config(f)
        c = model_config_from_dict(cfg["model"])
        assert c.hidden_size > 0


def test_unknown_model_key_is_an_error():
    cfg = tiny_cfg()
    cfg["model"]["not_a_key"] = 1
    with pytest.raises(ValueError):
        build_model(cfg)
    with pytest.raises(ValueError):
        build_model(tiny_cfg(attention_bias=True))


@pytest.mark.parametrize("mtype", MOE_TYPES + ["dense"])
def test_forward_shapes_and_outputs(mtype):
    model, cfg = build_model(tiny_cfg(mtype), seed=0)
    ids = batch()
    out = model(input_ids=ids, labels=ids, output_router_logits=True)
    assert out.loss.ndim == 0 and torch.isfinite(out.loss)
    if mtype == "dense":
        assert out.router_logits is None and out.aux_loss is None
    else:
        assert len(out.router_logits) == cfg.num_hidden_layers
        for r in out.router_logits:
            assert r.shape == (ids.numel(), cfg.num_experts) and r.dtype == torch.float32
        assert out.aux_loss is not None
    out2 = model(input_ids=ids)
    assert out2.logits.shape == (2, 16, 256) and out2.loss is None


def test_class_mapping_and_router_types():
    m, _ = build_model(tiny_cfg("standard_moe"))
    assert isinstance(m, StandardMoEModel) and not any(isinstance(x, DeepSeekRouter) for x in m.modules())
    m, _ = build_model(tiny_cfg("deepseek_standard_moe"))
    assert isinstance(m, DeepSeekStandardMoEModel)
    assert sum(isinstance(x, DeepSeekRouter) for x in m.modules()) == 2
    m, _ = build_model(tiny_cfg("global_moe"))
    assert isinstance(m, GlobalMoEForCausalLM)
    m, _ = build_model(tiny_cfg("deepseek_global_moe"))
    assert isinstance(m, DeepSeekGlobalMoEForCausalLM) and m._seq_aux_loss_coef == 1e-3


def test_global_bank_registered_once_and_names():
    m, cfg = build_model(tiny_cfg("global_moe"))
    names = [n for n, _ in m.named_parameters()]
    assert names.count("model.global_experts.gate_up_proj") == 1
    assert not any(".mlp.experts." in n for n in names)
    assert m.model.global_experts.gate_up_proj.shape == (16, 64, 64)
    assert m.model.global_experts.down_proj.shape == (16, 64, 32)
    for i in range(cfg.num_hidden_layers):
        assert f"model.layers.{i}.mlp.gate.weight" in names
    s, _ = build_model(tiny_cfg("standard_moe"))
    sn = dict(s.named_parameters())
    assert sn["model.layers.0.mlp.experts.gate_up_proj"].shape == (8, 64, 64)
    for key in ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight",
                "model.layers.0.self_attn.q_norm.weight", "model.layers.1.post_attention_layernorm.weight",
                "model.norm.weight", "lm_head.weight"]:
        assert key in sn
    d, _ = build_model(tiny_cfg("deepseek_standard_moe"))
    assert "model.layers.0.mlp.gate.expert_bias" in d.state_dict()
    assert "model.layers.0.mlp.gate.local_tokens_per_expert" not in d.state_dict()


def test_expert_parameter_parity_standard_vs_global():
    s, _ = build_model(tiny_cfg("standard_moe", num_experts=8))
    g, _ = build_model(tiny_cfg("global_moe", num_experts=16))  # 2 layers x 8
    ep = lambda m: sum(p.numel() for n, p in m.named_parameters() if "gate_up_proj" in n or "down_proj" in n)
    assert ep(s) == ep(g)


def test_param_counts_match_reference_shapes():
    # tiny BASELINE config: 39 389 952 parameters in the reference
    cfg = {"model": dict(type="standard_moe", vocab_size=151936, hidden_size=128, num_hidden_layers=2, head_dim=32,
                         num_attention_heads=4, num_key_value_heads=2, num_experts=8, num_experts_per_tok=2,
                         moe_intermediate_size=64, tie_word_embeddings=False)}
    with torch.device("meta"):
        m, _ = build_model(cfg)
    assert sum(p.numel() for p in m.parameters()) == 39_389_952


def test_tied_embeddings_share_storage():
    m, _ = build_model(tiny_cfg("standard_moe", tie_word_embeddings=True))
    assert m.lm_head.weight is m.model.embed_tokens.weight
    assert "lm_head.weight" not in [n for n, _ in m.named_parameters()]


def test_init_statistics_and_ce_at_init():
    m, _ = build_model(tiny_cfg("standard_moe", vocab_size=4096), seed=3)
    sd = dict(m.named_parameters())
    assert abs(sd["model.embed_tokens.weight"].std().item() - 0.02) < 2e-3
    assert abs(sd["model.layers.0.mlp.experts.down_proj"].std().item() - 0.02) < 2e-3
    assert abs(sd["model.layers.0.mlp.gate.weight"].std().item() - 0.02) < 4e-3
    assert torch.all(sd["model.norm.weight"] == 1) and torch.all(sd["model.layers.0.self_attn.q_norm.weight"] == 1)
    ids = batch(vocab=4096, B=2, S=64)
    out = m(input_ids=ids, labels=ids, output_router_logits=True)
    assert abs(out.ce_loss.item() - math.log(4096)) < 0.2
    assert abs(out.aux_loss.item() - 2.0) < 0.3  # uniform-ish routing gives top_k


def test_same_seed_same_weights_different_seed_differs():
    a, _ = build_model(tiny_cfg(), seed=5)
    b, _ = build_model(tiny_cfg(), seed=5)
    c, _ = build_model(tiny_cfg(), seed=6)
    assert all(torch.equal(p, q) for p, q in zip(a.parameters(), b.parameters()))
    assert not torch.equal(a.lm_head.weight, c.lm_head.weight)


@pytest.mark.parametrize("mtype", MOE_TYPES)
def test_loss_decomposition(mtype):
    m, cfg = build_model(tiny_cfg(mtype), seed=0)
    ids = batch()
    out = m(input_ids=ids, labels=ids, output_router_logits=True)
    expect = out.ce_loss + m.router_aux_loss_coef * out.aux_loss
    if m._seq_aux_loss_coef > 0:
        assert out.seq_aux_loss is not None
        expect = expect + m._seq_aux_loss_coef * out.seq_aux_loss
    assert torch.allclose(out.loss, expect, atol=1e-6)
    # the fixed aux loss is what the public function returns on the recorded scores
    ref = load_balancing_loss_func(out.router_logits, cfg.num_experts, cfg.num_experts_per_tok)
    assert torch.allclose(out.aux_loss, ref, atol=1e-6)


def test_aux_loss_zero_weighted_still_reported():
    m, _ = build_model(tiny_cfg("standard_moe", router_aux_loss_coef=0.0), seed=0)
    ids = batch()
    out = m(input_ids=ids, labels=ids, output_router_logits=True)
    assert out.aux_loss is not None and torch.allclose(out.loss, out.ce_loss)


@pytest.mark.parametrize("mtype", MOE_TYPES)
def test_gradients_reach_routers_and_experts(mtype):
    m, _ = build_model(tiny_cfg(mtype), seed=0)
    ids = batch()
    m(input_ids=ids, labels=ids, output_router_logits=True).loss.backward()
    for n, p in m.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n
        if "gate.weight" in n or "gate_up_proj" in n or "down_proj" in n:
            assert p.grad.abs().sum() > 0, n


def test_perturbing_global_expert_changes_loss_and_sgd_step_lowers_loss():
    m, _ = build_model(tiny_cfg("global_moe"), seed=0)
    ids = batch()
    l0 = m(input_ids=ids, labels=ids, output_router_logits=True).loss
    l0.backward()
    with torch.no_grad():
        for p in m.parameters():
            p -= 0.5 * p.grad
    l1 = m(input_ids=ids, labels=ids, output_router_logits=True).loss
    assert l1 < l0
    with torch.no_grad():
        m.model.global_experts.down_proj.add_(1.0)
    l2 = m(input_ids=ids, labels=ids, output_router_logits=True).loss
    assert abs(l2.item() - l1.item()) > 1e-4


def test_labels_are_shifted_once():
    m, _ = build_model(tiny_cfg("dense"), seed=0)
    ids = batch()
    out = m(input_ids=ids, labels=ids)
    logits = m(input_ids=ids).logits
    ref = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 256).float(), ids[:, 1:].reshape(-1))
    assert torch.allclose(out.loss, ref, atol=1e-5)
    lab = ids.clone()
    lab[:, 5:] = -100
    out2 = m(input_ids=ids, labels=lab)
    ref2 = torch.nn.functional.cross_entropy(logits[:, :4].reshape(-1, 256).float(), ids[:, 1:5].reshape(-1))
    assert torch.allclose(out2.loss, ref2, atol=1e-5)


def test_gradient_checkpointing_same_grads_and_counts_once():
    a, _ = build_model(tiny_cfg("deepseek_global_moe"), seed=0)
    b, _ = build_model(tiny_cfg("deepseek_global_moe"), seed=0)
    b.gradient_checkpointing_enable()
    ids = batch()
    a(input_ids=ids, labels=ids, output_router_logits=True).loss.backward()
    b(input_ids=ids, labels=ids, output_router_logits=True).loss.backward()
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6), n
    for ra, rb in zip(a.routers(), b.routers()):
        assert ra.local_tokens_per_expert.sum() == ids.numel() * 2
        assert torch.equal(ra.local_tokens_per_expert, rb.local_tokens_per_expert)


def test_generate_runs():
    m, _ = build_model(tiny_cfg("standard_moe"), seed=0)
    out = m.generate(batch(B=1, S=4), max_new_tokens=3)
    assert out.shape == (1, 7)


def test_sharded_optimizer_slices_tile_every_bucket():
    """The slice a rank owns in a gradient bucket (host arithmetic of `TrainEngine.owned_slice`) must be the
    one the reduce kernel reduces on that rank: whole float4 groups, ceil-divided over the ranks, disjoint,
    covering the bucket."""
    from moe_b200.models import build_model
    from moe_b200.parallel.engine import TrainEngine

    cfg = {"model": dict(type="dense", vocab_size=512, hidden_size=64, num_hidden_layers=3, head_dim=16,
                         num_attention_heads=4, num_key_value_heads=2, intermediate_size=128)}
    model, _ = build_model(cfg, seed=0, device="cpu")
    eng = TrainEngine(model, lr=1e-3)
    offs = [o for o in eng.layer_offsets() if o is not None]
    assert offs == sorted(offs) and len(offs) == 3
    eng.overlap = True  # plan as a multi-rank CUDA run would: one bucket per decoder layer
    buckets = eng.bucket_ranges()
    assert buckets[0][1] == eng.decay_end and buckets[-1][0] == 0
    assert all(a[0] == b[1] for a, b in zip(buckets, buckets[1:]))  # handed over from the top down, no gaps
    for world in (2, 3, 8):
        eng.world = world
        for lo, hi in buckets:
            n4 = (hi - lo) // 4
            per = -(-n4 // world)
            cover = []
            for r in range(world):
                a, b = eng.owned_slice(lo, hi, r)
                k_lo, k_hi = min(per * r, n4), min(per * r + per, n4)  # what the kernel computes
                assert (a, b) == (lo + 4 * k_lo, lo + 4 * k_hi)
                cover.append((a, b))
            assert cover[0][0] == lo and cover[-1][1] == lo + 4 * n4
            assert all(x[1] == y[0] for x, y in zip(cover, cover[1:]))
