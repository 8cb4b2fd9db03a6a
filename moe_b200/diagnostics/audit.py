"""Pipeline audit: eight end-to-end checks of a config before a long run
(`scripts/full_audit.py:27-443` of the reference), on synthetic data.

    python -m moe_b200.diagnostics.audit configs/bench/tiny_cpu.yaml [--device cpu]

1 parameter accounting  2 init statistics  3 CE at init = ln(vocab)  4 loss decomposition
5 gradients reach every parameter  6 optimizer groups / weight-decay rule  7 LR schedule end points
8 checkpoint round trip is bit exact.  Exit code 1 if any check fails.
"""
from __future__ import annotations

import argparse
import math
import sys
import tempfile

import torch

from ..data import SyntheticConfig, SyntheticTokenDataset
from ..models import build_model, load_config
from ..parallel.engine import is_no_decay
from ..trainer import Trainer
from ..utils.checkpoint import load_checkpoint, save_checkpoint
from ..utils.training import TrainingConfig, count_parameters, lr_factor


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("config")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seq", type=int, default=128)
    a = ap.parse_args(argv)
    cfg = load_config(a.config)
    tcfg = TrainingConfig.from_dict(dict(cfg["training"]))
    model, mcfg = build_model(cfg, seed=0, device=a.device)
    is_moe = cfg["model"]["type"] != "dense"
    results = []

    def check(name, ok, detail=""):
        results.append(ok)
        print(f"[{'PASS' if ok else 'FAIL'}] {name} {detail}")

    n = count_parameters(model)
    expert = sum(p.numel() for k, p in model.named_parameters() if "gate_up_proj" in k or "down_proj" in k)
    check("1 parameters", n["total"] == n["trainable"] > 0, f"total {n['total']:,} expert {expert:,}")
    sd = dict(model.named_parameters())
    emb = sd["model.embed_tokens.weight"].float().std().item()
    norms_one = all(bool((p == 1).all()) for k, p in sd.items() if "norm" in k)
    check("2 init", abs(emb - mcfg.initializer_range) < 0.1 * mcfg.initializer_range and norms_one, f"std(embed) {emb:.4f}")
    ds = iter(SyntheticTokenDataset(SyntheticConfig(mcfg.vocab_size, a.seq, 0)))
    ids = torch.stack([next(ds)["input_ids"] for _ in range(2)]).to(a.device)
    kw = {"output_router_logits": True} if is_moe else {}
    out = model(input_ids=ids, labels=ids, **kw)
    ce0, loss0 = float(out.ce_loss.detach()), float(out.loss.detach())
    check("3 CE at init", abs(ce0 - math.log(mcfg.vocab_size)) < 0.5,
          f"ce {ce0:.4f} ln V {math.log(mcfg.vocab_size):.4f}")
    expect = out.ce_loss.detach().float()
    if is_moe:
        expect = expect + model.router_aux_loss_coef * out.aux_loss.detach()
        if out.seq_aux_loss is not None:
            expect = expect + model._seq_aux_loss_coef * out.seq_aux_loss.detach()
    check("4 loss decomposition", abs(loss0 - float(expect.detach())) < 1e-4, f"loss {loss0:.5f}")
    out.loss.backward()
    missing = [k for k, p in model.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
    check("5 gradients", not missing, f"missing/non-finite: {missing[:3]}")
    model.zero_grad(set_to_none=True)
    decayed = {k for k, p in model.named_parameters() if not is_no_decay(k, p)}
    ok6 = "model.embed_tokens.weight" in decayed and all("norm" not in k for k in decayed)
    check("6 optimizer groups", ok6, f"{len(decayed)} decayed tensors")
    ok7 = lr_factor(0, tcfg) == (0.0 if tcfg.warmup_steps > 0 else lr_factor(0, tcfg)) and \
        abs(lr_factor(tcfg.warmup_steps, tcfg) - 1.0) < 1e-9 and \
        (tcfg.lr_scheduler == "constant" or abs(lr_factor(tcfg.max_steps, tcfg) - tcfg.min_lr_ratio) < 1e-9)
    check("7 LR schedule", ok7, f"{tcfg.lr_scheduler} warmup {tcfg.warmup_steps} max {tcfg.max_steps}")
    tr = Trainer(model, tcfg, is_moe=is_moe)
    tr.train_step({"input_ids": ids, "labels": ids})
    with tempfile.TemporaryDirectory() as d:
        path = save_checkpoint(tr, tr.global_step, d)
        before = [p.detach().clone() for p in model.parameters()]
        with torch.no_grad():
            for p in model.parameters():
                p.add_(1.0)
        step, _ = load_checkpoint(tr, path)
        same = all(torch.equal(p.detach(), q) for p, q in zip(model.parameters(), before))
        check("8 checkpoint round trip", same and step == 1)
    return 0 if all(results) else 1


if __name__ == "__main__":
    sys.exit(main())
