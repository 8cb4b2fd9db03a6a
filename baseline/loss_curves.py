#!/usr/bin/env python
"""Loss of every optimizer step, reference arm and this build, same config, seed and synthetic token stream.

    python baseline/loss_curves.py --steps 1000 --out curves.json [--config xs_standard] [--arms ours reference]

One GPU.  Both arms start from step 0 (no warm-up steps are discarded), use the learning-rate schedule of the
config and read the loss back every step; the reference arm is the installed reference package driven as in
`run_reference.py`.  Writes {"ours": {"loss": [...], "ce": [...], "aux": [...]}, "reference": {...}}.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def batches(n, B, S, V, seed):
    import torch

    g = torch.Generator().manual_seed(seed * 1000)
    return [torch.randint(0, V, (B, S), generator=g, dtype=torch.int64).pin_memory() for _ in range(n)]


def ours(cfg, data):
    import torch

    from moe_b200.models import build_model
    from moe_b200.trainer import Trainer
    from moe_b200.utils.training import TrainingConfig

    model, _ = build_model(cfg, seed=42, device="cuda:0")
    tr = Trainer(model, TrainingConfig.from_dict(cfg["training"]), cuda_graph=True)
    out = {"loss": [], "ce": [], "aux": []}
    for b in data:
        r = tr.train_step({"input_ids": b, "labels": b})
        vals = torch.stack([r.loss.float(), r.ce_loss.float(), r.aux_loss.float()]).tolist()
        for k, v in zip(("loss", "ce", "aux"), vals):
            out[k].append(round(v, 5))
    return out


def reference(cfg, data):
    import torch

    import run_reference as rr

    torch.manual_seed(42)
    model, mcfg, tcfg, build_optimizer, build_lr_scheduler, get_grad_norm, liger, impl = rr._build(
        cfg, os.path.join(ROOT, "baseline", "_ref"))
    model = model.to("cuda:0").train()
    opt = build_optimizer(model, tcfg)
    sched = build_lr_scheduler(opt, tcfg)
    coef = float(cfg["model"].get("router_aux_loss_coef", 0.001))
    out = {"loss": [], "ce": [], "aux": [], "stack": f"liger {liger}; experts {impl}"}
    for b in data:
        ids = b.cuda(non_blocking=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            o = model(input_ids=ids, labels=ids, output_router_logits=True)
        o.loss.backward()
        get_grad_norm(model)
        torch.nn.utils.clip_grad_norm_(model.parameters(), tcfg.max_grad_norm)
        opt.step()
        opt.zero_grad()
        sched.step()
        loss, aux = float(o.loss), float(o.aux_loss)
        out["loss"].append(round(loss, 5))
        out["aux"].append(round(aux, 5))
        out["ce"].append(round(loss - coef * aux, 5))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--config", default="xs_standard")
    ap.add_argument("--out", default="curves.json")
    ap.add_argument("--arms", nargs="+", default=["ours", "reference"])
    a = ap.parse_args()
    import yaml

    with open(os.path.join(ROOT, "configs", "bench", f"{a.config}.yaml")) as f:
        cfg = yaml.safe_load(f)
    B, S, V = cfg["training"]["batch_size"], cfg["data"]["seq_len"], cfg["model"]["vocab_size"]
    data = batches(a.steps, B, S, V, cfg["data"].get("seed", 0))
    res = {"config": a.config, "steps": a.steps}
    if os.path.exists(a.out):
        with open(a.out) as f:
            res.update(json.load(f))
    for arm in a.arms:
        res[arm] = ours(cfg, data) if arm == "ours" else reference(cfg, data)
        with open(a.out, "w") as f:
            json.dump(res, f)
        print(arm, "first", res[arm]["loss"][:3], "last", res[arm]["loss"][-3:], flush=True)


if __name__ == "__main__":
    main()
