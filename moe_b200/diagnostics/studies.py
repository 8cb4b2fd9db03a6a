"""Research diagnostics of the reference's `scripts/` folder as sub-commands on one harness.

    python -m moe_b200.diagnostics.studies compare-long  A.yaml B.yaml [C.yaml] --steps 1000 --csv out.csv
    python -m moe_b200.diagnostics.studies hidden-states STANDARD.yaml GLOBAL.yaml
    python -m moe_b200.diagnostics.studies identical-loss STANDARD.yaml GLOBAL.yaml
    python -m moe_b200.diagnostics.studies seed-vs-arch   STANDARD.yaml GLOBAL.yaml --steps 50
    python -m moe_b200.diagnostics.studies dense-vs-moe   DENSE.yaml STANDARD.yaml GLOBAL.yaml
    python -m moe_b200.diagnostics.studies high-lr        STANDARD.yaml GLOBAL.yaml --lrs 1e-2 1e-1 1.0
    python -m moe_b200.diagnostics.studies kernel-effect  STANDARD.yaml GLOBAL.yaml      (CUDA only)
    python -m moe_b200.diagnostics.studies scale-check    configs/bench/l_standard.yaml --layers 2
    python -m moe_b200.diagnostics.studies real-vs-random STANDARD.yaml --data_dir data/parquet

Reference scripts, in the same order: `compare_1000_steps.py:26-83`, `first_principles.py:58-122` and
`test_hidden_states.py:23-62`, `diagnose_identical_loss.py:94-272`, `test_seed_vs_arch.py`,
`test_dense_vs_moe.py`, `test_high_lr.py`, `test_liger_effect.py` (here: kernels against the plain-PyTorch
ops instead of Liger on/off), `test_l_scale.py`, `test_real_vs_random_data.py`.  All default to the synthetic
token stream so that they run offline; every function returns its numbers as a dict for programmatic use.
"""
from __future__ import annotations

import argparse
import time

import torch

from . import harness as H


def _name(c) -> str:
    return c["model"]["type"] if isinstance(c, dict) else str(c).split("/")[-1].replace(".yaml", "")


def compare_long(configs, steps=1000, every=50, csv=None, **kw) -> dict:
    runs = [H.run_steps(c, steps, **kw)["rows"] for c in configs]
    names = [_name(c) for c in configs]
    print("step  " + "  ".join(f"{n[:18]:>18s} ce" for n in names))
    for i in range(0, steps, max(1, every)):
        j = min(i + every, steps)
        print(f"{j:5d} " + "  ".join(f"{sum(r['ce'] for r in run[i:j]) / (j - i):21.4f}" for run in runs))
    out = {f"mean_abs_ce_diff[{n}-{names[0]}]": H.mean_abs_diff(runs[0], r) for n, r in zip(names[1:], runs[1:])}
    for k, v in out.items():
        print(f"{k} = {v:.5f}")
    if csv:
        H.write_csv(csv, names, runs)
    return {"names": names, "runs": runs, **out}


def hidden_states(cfg_a, cfg_b, seed=42, other_seed=123, device="cpu", batch=2, seq=64, train_steps=0, **kw) -> dict:
    """Layer-wise cosine similarity of the residual stream: architecture A vs B (same seed), and A vs A with
    another seed, on the same tokens; plus the similarity of the output logits."""
    def prep(cfg, s):
        if train_steps:
            return H.run_steps(cfg, train_steps, seed=s, data_seed=seed, device=device, batch=batch, seq=seq)["trainer"].model
        return H.make_trainer(cfg, s, device)[0].model

    a, b, a2 = prep(cfg_a, seed), prep(cfg_b, seed), prep(cfg_a, other_seed)
    ids = next(H.batches(H.as_config(cfg_a), batch, seq, seed + 1)).to(device)
    ha, hb, ha2 = (H.layer_hidden_states(m, ids) for m in (a, b, a2))
    arch = [H.cosine(x, y) for x, y in zip(ha, hb)]
    sd = [H.cosine(x, y) for x, y in zip(ha, ha2)]
    with torch.no_grad():
        la, lb, la2 = (m(input_ids=ids, output_router_logits=False).logits.float() for m in (a, b, a2))
    res = {"layer_cos_arch": arch, "layer_cos_seed": sd, "logit_cos_arch": H.cosine(la, lb),
           "logit_cos_seed": H.cosine(la, la2)}
    print("layer   cos(A, B same seed)   cos(A, A other seed)")
    for i, (x, y) in enumerate(zip(arch, sd)):
        print(f"{i:5d} {x:21.4f} {y:22.4f}")
    print(f"logits {res['logit_cos_arch']:21.4f} {res['logit_cos_seed']:22.4f}")
    return res


def identical_loss(cfg_a, cfg_b, seed=42, device="cpu", batch=2, seq=64, steps=3, **kw) -> dict:
    """Five checks on why two layouts may give near-identical loss curves."""
    res = {}
    ta, ca, _ = H.make_trainer(cfg_a, seed, device)
    tb, cb, _ = H.make_trainer(cfg_b, seed, device)
    ids = next(H.batches(ca, batch, seq, seed)).to(device)
    ea = {n: p for n, p in ta.model.named_parameters() if "gate_up_proj" in n or "down_proj" in n}
    eb = {n: p for n, p in tb.model.named_parameters() if "gate_up_proj" in n or "down_proj" in n}
    res["1_expert_param_counts"] = (sum(p.numel() for p in ea.values()), sum(p.numel() for p in eb.values()))
    res["1_expert_tensor_names_differ"] = set(ea) != set(eb)
    sa, sb = H.layer_hidden_states(ta.model, ids), H.layer_hidden_states(tb.model, ids)
    res["2_layer_output_cos"] = [H.cosine(x, y) for x, y in zip(sa, sb)]
    with torch.no_grad():
        full = float(ta.model(input_ids=ids, labels=ids, output_router_logits=True).ce_loss)
    abl, _, _ = H.make_trainer(cfg_a, seed, device, mutate=H.zero_moe_output)
    with torch.no_grad():
        no_ffn = float(abl.model(input_ids=ids, labels=ids, output_router_logits=False).loss)
    res["3_ce_full_vs_without_experts"] = (full, no_ffn)
    before = {n: p.detach().float().clone() for n, p in ea.items()}
    rw = {n: p.detach().float().clone() for n, p in ta.model.named_parameters() if n.endswith("mlp.gate.weight")}
    for _ in range(steps):
        ta.train_step({"input_ids": ids, "labels": ids})
    cur = dict(ta.model.named_parameters())
    res["4_router_weight_change"] = {n: float((cur[n].detach().float() - w).norm()) for n, w in rw.items()}
    res["5_expert_weight_change"] = {n: float((cur[n].detach().float() - w).norm()) for n, w in before.items()}
    for k, v in res.items():
        print(f"{k}: {v}")
    return res


def seed_vs_arch(cfg_a, cfg_b, steps=50, seed=42, other_seed=7, **kw) -> dict:
    """Does another seed (same layout) move the curve more than another layout (same seed)?"""
    a1 = H.run_steps(cfg_a, steps, seed=seed, data_seed=seed, **kw)["rows"]
    a2 = H.run_steps(cfg_a, steps, seed=other_seed, data_seed=seed, **kw)["rows"]
    b1 = H.run_steps(cfg_b, steps, seed=seed, data_seed=seed, **kw)["rows"]
    res = {"seed_diff": H.mean_abs_diff(a1, a2), "arch_diff": H.mean_abs_diff(a1, b1)}
    print(f"mean |ce| difference: other seed {res['seed_diff']:.5f}   other layout {res['arch_diff']:.5f}")
    return res


def dense_vs_moe(configs, steps=50, **kw) -> dict:
    """Dense, the MoE layouts, and the first MoE config with its expert blocks zeroed."""
    names = [_name(c) for c in configs]
    runs = [H.run_steps(c, steps, **kw)["rows"] for c in configs]
    moe = next((c for c in configs if H.as_config(c)["model"]["type"] != "dense"), configs[0])
    runs.append(H.run_steps(moe, steps, mutate=H.zero_moe_output, **kw)["rows"])
    names.append(_name(moe) + "-no-experts")
    res = {n: sum(r["ce"] for r in run[-max(1, steps // 5):]) / max(1, steps // 5) for n, run in zip(names, runs)}
    for n, v in res.items():
        print(f"{n:>32s}: mean ce over the last fifth = {v:.4f}")
    return res


def high_lr(cfg_a, cfg_b, lrs=(1e-2, 1e-1, 1.0), steps=50, **kw) -> dict:
    res = {}
    for lr in lrs:
        a = H.run_steps(cfg_a, steps, lr=lr, warmup=0, **kw)["rows"]
        b = H.run_steps(cfg_b, steps, lr=lr, warmup=0, **kw)["rows"]
        res[lr] = {"diff": H.mean_abs_diff(a, b), "final_a": a[-1]["ce"], "final_b": b[-1]["ce"]}
        print(f"lr {lr:g}: mean |ce_a - ce_b| = {res[lr]['diff']:.5f}  final {a[-1]['ce']:.4f} / {b[-1]['ce']:.4f}")
    return res


def kernel_effect(cfg_a, cfg_b, steps=30, **kw) -> dict:
    """Layout difference measured on the sm_100a kernels and on the plain-PyTorch ops of the same device."""
    from .. import ops

    kw = dict(kw, device="cuda")
    res = {}
    for label, ctx in (("kernels", None), ("plain", ops.force_oracle)):
        if ctx is None:
            a, b = (H.run_steps(c, steps, **kw)["rows"] for c in (cfg_a, cfg_b))
        else:
            with ctx():
                a, b = (H.run_steps(c, steps, **kw)["rows"] for c in (cfg_a, cfg_b))
        res[label] = {"arch_diff": H.mean_abs_diff(a, b), "rows_a": a}
        print(f"{label:>8s}: mean |ce(A) - ce(B)| = {res[label]['arch_diff']:.5f}")
    res["kernel_vs_plain"] = H.mean_abs_diff(res["kernels"]["rows_a"], res["plain"]["rows_a"])
    print(f"same layout, kernels vs plain ops: mean |ce| difference {res['kernel_vs_plain']:.5f}")
    return res


def scale_check(cfg, layers=None, steps=2, device="cpu", **kw) -> dict:
    """Build a (possibly shortened) large config with activation recomputation, run a step, report time/memory."""
    c = H.as_config(cfg)
    if layers:
        c["model"]["num_hidden_layers"] = layers
    c.setdefault("training", {})["gradient_checkpointing"] = True
    t0 = time.perf_counter()
    out = H.run_steps(c, steps, device=device, **kw)
    if device == "cuda":
        torch.cuda.synchronize()
    n = sum(p.numel() for p in out["trainer"].model.parameters())
    res = {"params": n, "seconds_per_step": (time.perf_counter() - t0) / steps, "ce": out["rows"][-1]["ce"],
           "peak_memory_gb": torch.cuda.max_memory_allocated() / 2**30 if device == "cuda" else None}
    print(res)
    return res


def real_vs_random(cfg, data_dir, steps=50, **kw) -> dict:
    real = H.run_steps(cfg, steps, data_dir=data_dir, **kw)["rows"]
    rand = H.run_steps(cfg, steps, **kw)["rows"]
    res = {"final_ce_real": real[-1]["ce"], "final_ce_random": rand[-1]["ce"]}
    print(f"final ce: corpus {res['final_ce_real']:.4f}   uniform random tokens {res['final_ce_random']:.4f}")
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("study", choices=["compare-long", "hidden-states", "identical-loss", "seed-vs-arch", "dense-vs-moe",
                                      "high-lr", "kernel-effect", "scale-check", "real-vs-random"])
    ap.add_argument("configs", nargs="+")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--lr", type=float, default=None)
    ap.add_argument("--lrs", type=float, nargs="*", default=[1e-2, 1e-1, 1.0])
    ap.add_argument("--every", type=int, default=50)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--data_dir", default=None)
    a = ap.parse_args(argv)
    kw = dict(seed=a.seed, device=a.device, batch=a.batch, seq=a.seq)
    st = {} if a.steps is None else {"steps": a.steps}
    c = a.configs
    if a.study == "compare-long":
        return compare_long(c, every=a.every, csv=a.csv, lr=a.lr, data_dir=a.data_dir, **st, **kw)
    if a.study == "hidden-states":
        return hidden_states(c[0], c[1], seed=a.seed, device=a.device, batch=a.batch or 2, seq=a.seq or 64,
                             train_steps=a.steps or 0)
    if a.study == "identical-loss":
        return identical_loss(c[0], c[1], seed=a.seed, device=a.device, batch=a.batch or 2, seq=a.seq or 64)
    if a.study == "seed-vs-arch":
        return seed_vs_arch(c[0], c[1], device=a.device, batch=a.batch, seq=a.seq, lr=a.lr, **st)
    if a.study == "dense-vs-moe":
        return dense_vs_moe(c, lr=a.lr, **st, **kw)
    if a.study == "high-lr":
        return high_lr(c[0], c[1], lrs=a.lrs, **st, **kw)
    if a.study == "kernel-effect":
        return kernel_effect(c[0], c[1], seed=a.seed, batch=a.batch, seq=a.seq, **st)
    if a.study == "scale-check":
        return scale_check(c[0], layers=a.layers, seed=a.seed, device=a.device, batch=a.batch, seq=a.seq, **st)
    return real_vs_random(c[0], a.data_dir, **st, **kw)


if __name__ == "__main__":
    main()
