"""Tiny standard-vs-global diagnostic (`scripts/debug_tiny_global_vs_perlayer.py:29-245`): builds a
small standard model and a global model with the same backbone seed, checks that the two differ
only in where the experts live (parameter parity, distinct outputs, gradients reaching the shared
bank from every layer) and prints per-layer routing statistics after a few steps.

    python -m moe_b200.diagnostics.tiny_global_vs_perlayer [--device cpu] [--steps 10]
"""
from __future__ import annotations

import argparse

import torch

from ..models import build_model
from ..utils.routing_stats import compute_routing_stats


def tiny(mtype: str, experts: int) -> dict:
    return {"model": dict(type=mtype, vocab_size=512, hidden_size=128, num_hidden_layers=4, head_dim=32,
                          num_attention_heads=4, num_key_value_heads=2, num_experts=experts, num_experts_per_tok=2,
                          moe_intermediate_size=64, router_aux_loss_coef=0.01)}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=10)
    a = ap.parse_args(argv)
    std, _ = build_model(tiny("standard_moe", 4), seed=0, device=a.device)
    glb, _ = build_model(tiny("global_moe", 16), seed=0, device=a.device)
    ep = lambda m: sum(p.numel() for n, p in m.named_parameters() if "gate_up_proj" in n or "down_proj" in n)
    print(f"expert params: standard {ep(std):,}  global {ep(glb):,}  (equal: {ep(std) == ep(glb)})")
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (4, 64), generator=g).to(a.device)
    for name, m in (("standard", std), ("global", glb)):
        opt = torch.optim.SGD(m.parameters(), lr=0.5)
        for step in range(a.steps):
            out = m(input_ids=ids, labels=ids, output_router_logits=True)
            opt.zero_grad()
            out.loss.backward()
            if step == 0:
                bank = [p for n, p in m.named_parameters() if "gate_up_proj" in n]
                print(f"[{name}] step 0 loss {float(out.loss):.4f}; banks {len(bank)}; "
                      f"bank grad norms {[round(float(p.grad.float().norm()), 4) for p in bank]}")
            opt.step()
        stats = compute_routing_stats(out.router_logits, 2, is_global=name == "global")
        keys = [k for k in stats if k.endswith("load_imbalance") or "cross_layer_sim_mean" in k]
        print(f"[{name}] final loss {float(out.loss):.4f}  " + "  ".join(f"{k.split('/')[-1]}={stats[k]:.3f}" for k in keys))


if __name__ == "__main__":
    main()
