"""Smoke runs of the research diagnostics on tiny CPU models: every study returns sensible numbers."""
import math

import pytest

from helpers import tiny_cfg
from moe_b200.diagnostics import studies as S

STD, GLB, DENSE = tiny_cfg("standard_moe"), tiny_cfg("global_moe"), tiny_cfg("dense")
KW = dict(device="cpu", batch=2, seq=16)


def test_compare_long_and_csv(tmp_path):
    out = S.compare_long([STD, GLB], steps=6, every=3, csv=str(tmp_path / "c.csv"), **KW)
    assert len(out["runs"]) == 2 and len(out["runs"][0]) == 6
    assert all(math.isfinite(r["ce"]) for run in out["runs"] for r in run)
    assert (tmp_path / "c.csv").read_text().count("\n") == 7


def test_hidden_states_same_seed_shares_the_backbone_start():
    res = S.hidden_states(STD, GLB, device="cpu", batch=2, seq=16)
    assert res["layer_cos_arch"][0] > 0.999  # same seed: identical embeddings
    assert res["layer_cos_seed"][0] < 0.5    # another seed: unrelated embeddings
    assert len(res["layer_cos_arch"]) == 3   # embedding + two layers


def test_identical_loss_checks():
    res = S.identical_loss(STD, GLB, device="cpu", batch=2, seq=16, steps=2)
    assert res["1_expert_tensor_names_differ"]
    assert all(v > 0 for v in res["4_router_weight_change"].values())
    assert all(v > 0 for v in res["5_expert_weight_change"].values())
    full, ablated = res["3_ce_full_vs_without_experts"]
    assert math.isfinite(full) and math.isfinite(ablated)


def test_seed_vs_arch_dense_vs_moe_high_lr():
    r = S.seed_vs_arch(STD, GLB, steps=4, **KW)
    assert r["seed_diff"] >= 0 and r["arch_diff"] >= 0
    d = S.dense_vs_moe([DENSE, STD, GLB], steps=5, **KW)
    assert any(k.endswith("-no-experts") for k in d) and len(d) == 4
    h = S.high_lr(STD, GLB, lrs=(1e-2, 1e-1), steps=3, **KW)
    assert set(h) == {1e-2, 1e-1}


def test_scale_check_runs_with_recomputation():
    r = S.scale_check(tiny_cfg("standard_moe", num_hidden_layers=4), layers=2, steps=1, device="cpu", batch=2, seq=16)
    assert r["params"] > 0 and r["seconds_per_step"] > 0 and math.isfinite(r["ce"])


def test_cli_dispatch():
    import yaml, tempfile, os

    with tempfile.TemporaryDirectory() as d:
        paths = []
        for i, c in enumerate((STD, GLB)):
            p = os.path.join(d, f"c{i}.yaml")
            with open(p, "w") as f:
                yaml.safe_dump({**c, "training": {"learning_rate": 1e-3, "batch_size": 2, "max_steps": 10},
                                "data": {"seq_len": 16, "source": "synthetic"}}, f)
            paths.append(p)
        out = S.main(["seed-vs-arch", *paths, "--steps", "2", "--device", "cpu"])
        assert "seed_diff" in out
