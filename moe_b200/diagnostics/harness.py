"""Shared pieces of the research diagnostics: load a config (file path or dict), build model + trainer with
overrides, produce batches (synthetic uniform tokens, or a parquet directory with a tokenizer), run steps and
collect per-step numbers.  Everything works on CPU (plain PyTorch ops) and on a B200 (kernels)."""
from __future__ import annotations

import copy
import csv
from typing import Callable, Iterator

import torch

from ..data import SyntheticConfig, SyntheticTokenDataset
from ..models import build_model, load_config
from ..trainer import Trainer
from ..utils.bias_update import bias_alpha_schedule, update_expert_biases
from ..utils.training import TrainingConfig


def as_config(cfg) -> dict:
    return copy.deepcopy(cfg) if isinstance(cfg, dict) else load_config(cfg)


def batches(cfg: dict, batch: int, seq: int, seed: int, data_dir: str | None = None,
            tokenizer_name: str | None = None) -> Iterator[torch.Tensor]:
    """`[batch, seq]` token ids: the seeded synthetic stream, or windows of a parquet corpus."""
    vocab = cfg["model"]["vocab_size"]
    if data_dir is None:
        ds = iter(SyntheticTokenDataset(SyntheticConfig(vocab, seq, seed)))
    else:
        from transformers import AutoTokenizer

        from ..data import DataConfig, StatefulParquetDataset

        tok = AutoTokenizer.from_pretrained(tokenizer_name or cfg.get("data", {}).get("tokenizer_name", "gpt2"))
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        ds = iter(StatefulParquetDataset(DataConfig(data_dir=data_dir, seq_len=seq), tok, rank=0, world_size=1))
    while True:
        yield torch.stack([next(ds)["input_ids"] for _ in range(batch)])


def make_trainer(cfg, seed: int = 42, device: str = "cpu", lr: float | None = None, batch: int | None = None,
                 warmup: int | None = None, mutate: Callable | None = None):
    cfg = as_config(cfg)
    t = dict(cfg.get("training", {}))
    t.setdefault("learning_rate", 1e-3)
    t.setdefault("max_steps", 10_000)
    if lr is not None:
        t["learning_rate"] = lr
    if batch is not None:
        t["batch_size"] = batch
    if warmup is not None:
        t["warmup_steps"] = warmup
    t["gradient_accumulation"] = 1
    if "warmup_steps" not in t:
        t["warmup_steps"] = 0
    known = set(TrainingConfig.__dataclass_fields__)
    tcfg = TrainingConfig(**{k: v for k, v in t.items() if k in known})  # a study may pass a partial section
    model, mcfg = build_model(cfg, seed=seed, device=device)
    if mutate is not None:
        mutate(model)
    tr = Trainer(model, tcfg, is_moe=cfg["model"]["type"] != "dense")
    return tr, cfg, tcfg


def run_steps(cfg, steps: int, *, seed: int = 42, data_seed: int | None = None, device: str = "cpu",
              lr: float | None = None, batch: int | None = None, seq: int | None = None, warmup: int | None = None,
              data_dir: str | None = None, mutate: Callable | None = None, on_step: Callable | None = None) -> dict:
    """Train `steps` optimizer steps.  Returns {"rows": per-step dicts, "trainer": Trainer, "cfg": dict}."""
    tr, cfg, tcfg = make_trainer(cfg, seed, device, lr, batch, warmup, mutate)
    seq = seq or cfg.get("data", {}).get("seq_len", 256)
    it = batches(cfg, tcfg.batch_size, seq, seed if data_seed is None else data_seed, data_dir)
    mtype = cfg["model"]["type"]
    rate = cfg["model"].get("bias_update_rate", 0.0) or 0.0
    rows = []
    for step in range(steps):
        ids = next(it)
        r = tr.train_step({"input_ids": ids, "labels": ids})
        if rate > 0:
            is_global = "global" in mtype
            alpha = bias_alpha_schedule(step) if (is_global and cfg["model"].get("bias_interpolation")) else 0.0
            update_expert_biases(tr.model, rate, None, is_global=is_global, alpha=alpha)
        row = {"step": step + 1, "loss": float(r.loss),
               "ce": float(r.ce_loss) if r.ce_loss is not None else float(r.loss),
               "aux": float(r.aux_loss) if r.aux_loss is not None else 0.0, "gnorm": float(r.grad_norm)}
        rows.append(row)
        if on_step is not None:
            on_step(step, tr, r, ids)
    return {"rows": rows, "trainer": tr, "cfg": cfg}


def mean_abs_diff(a: list[dict], b: list[dict], key: str = "ce", skip: int = 0) -> float:
    d = [abs(x[key] - y[key]) for x, y in zip(a[skip:], b[skip:])]
    return sum(d) / max(len(d), 1)


def write_csv(path: str, names: list[str], runs: list[list[dict]]) -> None:
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["step"] + [f"{n}_{k}" for n in names for k in ("loss", "ce", "aux", "gnorm")])
        for i in range(len(runs[0])):
            w.writerow([runs[0][i]["step"]] + [r[i][k] for r in runs for k in ("loss", "ce", "aux", "gnorm")])


def layer_hidden_states(model, ids: torch.Tensor) -> list[torch.Tensor]:
    """Residual stream after the embedding and after every decoder layer (captured with forward hooks)."""
    states: list[torch.Tensor] = []
    hooks = [model.model.embed_tokens.register_forward_hook(lambda m, i, o: states.append(o.detach().float()))]
    for layer in model.model.layers:
        hooks.append(layer.register_forward_hook(lambda m, i, o: states.append(o[0].detach().float())))
    with torch.no_grad():
        model(input_ids=ids, output_router_logits=False)
    for h in hooks:
        h.remove()
    return states


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0))


def zero_moe_output(model) -> None:
    """Ablation: every MoE / MLP block returns zeros (the model becomes attention-only)."""
    for layer in model.model.layers:
        def fwd(x, global_experts=None, _m=layer.mlp):
            return torch.zeros_like(x), None
        layer.mlp.forward = fwd
