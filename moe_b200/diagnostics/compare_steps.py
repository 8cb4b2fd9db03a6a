"""Step-by-step loss comparison of several configs under identical seed, data and optimizer
(`scripts/compare_training_steps.py:47-144`, `scripts/compare_1000_steps.py:26-83` of the reference).

    python -m moe_b200.diagnostics.compare_steps configs/bench/tiny_cpu.yaml other.yaml --steps 20 [--device cpu]

Prints one row per step with every config's total / ce / aux loss and the difference to the first
config, then the mean absolute difference.  Data: the synthetic uniform-token stream of the seed.
"""
from __future__ import annotations

import argparse

import torch

from ..data import SyntheticConfig, SyntheticTokenDataset
from ..models import build_model, load_config
from ..trainer import Trainer
from ..utils.bias_update import bias_alpha_schedule, update_expert_biases
from ..utils.training import TrainingConfig


def run_config(path: str, steps: int, device: str, seed: int, batch: int | None, seq: int | None) -> list[dict]:
    cfg = load_config(path)
    t = dict(cfg["training"])
    if batch:
        t["batch_size"] = batch
    tcfg = TrainingConfig.from_dict(t)
    seq = seq or cfg.get("data", {}).get("seq_len", 256)
    model, mcfg = build_model(cfg, seed=seed, device=device)
    mtype = cfg["model"]["type"]
    tr = Trainer(model, tcfg, is_moe=mtype != "dense")
    ds = iter(SyntheticTokenDataset(SyntheticConfig(cfg["model"]["vocab_size"], seq, seed)))
    rate = cfg["model"].get("bias_update_rate", 0.0) or 0.0
    rows = []
    for step in range(steps):
        ids = torch.stack([next(ds)["input_ids"] for _ in range(tcfg.batch_size)])
        r = tr.train_step({"input_ids": ids, "labels": ids})
        if rate > 0:
            is_global = "global" in mtype
            alpha = bias_alpha_schedule(step) if (is_global and cfg["model"].get("bias_interpolation")) else 0.0
            update_expert_biases(model, rate, None, is_global=is_global, alpha=alpha)
        rows.append({"loss": float(r.loss), "ce": float(r.ce_loss) if r.ce_loss is not None else float("nan"),
                     "aux": float(r.aux_loss) if r.aux_loss is not None else 0.0, "gnorm": float(r.grad_norm)})
    return rows


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("configs", nargs="+")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--seq", type=int, default=None)
    a = ap.parse_args(argv)
    runs = [run_config(c, a.steps, a.device, a.seed, a.batch, a.seq) for c in a.configs]
    names = [c.split("/")[-1].replace(".yaml", "") for c in a.configs]
    print("step  " + "  ".join(f"{n[:22]:>22s}(loss/ce/aux)" for n in names) + "   d_ce vs first")
    diffs = [[] for _ in runs]
    for s in range(a.steps):
        cells = [f"{r[s]['loss']:8.4f}/{r[s]['ce']:8.4f}/{r[s]['aux']:7.4f}" for r in runs]
        d = [r[s]["ce"] - runs[0][s]["ce"] for r in runs]
        for i, x in enumerate(d):
            diffs[i].append(abs(x))
        print(f"{s + 1:4d}  " + "  ".join(f"{c:>35s}" for c in cells) + "   " + " ".join(f"{x:+.4f}" for x in d[1:]))
    for n, d in zip(names[1:], diffs[1:]):
        print(f"mean |ce({n}) - ce({names[0]})| = {sum(d) / len(d):.5f}")


if __name__ == "__main__":
    main()
