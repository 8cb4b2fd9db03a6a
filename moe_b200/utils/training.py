"""Training utilities with the reference's public names (`src/utils/training.py:11-95`):
`TrainingConfig`, `build_optimizer`, `build_lr_scheduler`, `count_parameters`, `get_grad_norm`.

The optimizer / scheduler classes returned here are small stand-alone objects (no Accelerate);
the training loop proper uses `moe_b200.parallel.engine.TrainEngine`, which applies the same
update rule over flat buffers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import oracle
from ..parallel.engine import is_no_decay


@dataclass
class TrainingConfig:
    learning_rate: float = 3e-4
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler: str = "cosine"  # cosine | linear | constant
    warmup_steps: int = 2000
    max_steps: int = 100_000
    min_lr_ratio: float = 0.1
    batch_size: int = 4  # per GPU
    gradient_accumulation: int = 4
    mixed_precision: str = "bf16"
    gradient_checkpointing: bool = False
    log_every: int = 10
    routing_log_every: int = 50
    save_every: int = 5000
    output_dir: str = "./outputs"
    wandb_project: str | None = "moe-experiments"
    wandb_run_name: str | None = None

    @classmethod
    def from_dict(cls, d: dict) -> "TrainingConfig":
        known = set(cls.__dataclass_fields__)
        unknown = set(d) - known
        if unknown:
            raise ValueError(f"unknown training config keys: {sorted(unknown)}")
        for req in ("learning_rate", "weight_decay", "max_grad_norm", "lr_scheduler", "warmup_steps", "max_steps",
                    "min_lr_ratio", "batch_size", "gradient_accumulation", "mixed_precision", "log_every",
                    "save_every", "output_dir"):
            if req not in d:
                raise ValueError(f"training.{req} is required")
        if d["lr_scheduler"] not in ("cosine", "linear", "constant"):
            raise ValueError(f"unknown lr_scheduler {d['lr_scheduler']!r}")
        return cls(**d)


def lr_factor(step: int, config: TrainingConfig) -> float:
    """Multiplier on the base LR at optimizer step `step` (linear warm-up, then cosine / linear / constant)."""
    warmup, total, min_ratio = config.warmup_steps, config.max_steps, config.min_lr_ratio
    if step < warmup:
        return step / max(1, warmup)
    if config.lr_scheduler == "constant":
        return 1.0
    progress = min((step - warmup) / max(1, total - warmup), 1.0)
    if config.lr_scheduler == "cosine":
        return min_ratio + 0.5 * (1 - min_ratio) * (1 + math.cos(math.pi * progress))
    if config.lr_scheduler == "linear":
        return max(min_ratio, 1.0 - progress * (1 - min_ratio))
    return 1.0


class AdamW:
    """Decoupled-weight-decay Adam over parameter groups; same arithmetic as `torch.optim.AdamW`."""

    def __init__(self, param_groups, lr: float, betas=(0.9, 0.95), eps: float = 1e-8):
        self.param_groups = []
        for g in param_groups:
            g = dict(g)
            g.setdefault("lr", lr)
            g.setdefault("initial_lr", g["lr"])
            g.setdefault("betas", betas)
            g.setdefault("eps", eps)
            g.setdefault("weight_decay", 0.0)
            g["params"] = list(g["params"])
            self.param_groups.append(g)
        self.state: dict = {}
        self._step = 0

    def zero_grad(self, set_to_none: bool = True) -> None:
        for g in self.param_groups:
            for p in g["params"]:
                if set_to_none:
                    p.grad = None
                elif p.grad is not None:
                    p.grad.zero_()

    @torch.no_grad()
    def step(self) -> None:
        self._step += 1
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state.setdefault(p, {"exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)})
                oracle.adamw_step_(p, p.grad, st["exp_avg"], st["exp_avg_sq"], lr=g["lr"], beta1=b1, beta2=b2,
                                   eps=g["eps"], weight_decay=g["weight_decay"], step=self._step)

    def state_dict(self) -> dict:
        flat = []
        for g in self.param_groups:
            for p in g["params"]:
                st = self.state.get(p)
                flat.append(None if st is None else {k: v.clone() for k, v in st.items()})
        return {"step": self._step, "state": flat, "lrs": [g["lr"] for g in self.param_groups]}

    def load_state_dict(self, sd: dict) -> None:
        self._step = sd["step"]
        it = iter(sd["state"])
        for g, lr in zip(self.param_groups, sd["lrs"]):
            g["lr"] = lr
            for p in g["params"]:
                st = next(it)
                if st is not None:
                    self.state[p] = {k: v.clone() for k, v in st.items()}


class LambdaLR:
    """`lr = initial_lr * fn(step)`; `step()` once per optimizer step."""

    def __init__(self, optimizer, fn):
        self.optimizer, self.fn = optimizer, fn
        self.last_epoch = 0
        self._apply()

    def _apply(self) -> None:
        for g in self.optimizer.param_groups:
            g["lr"] = g["initial_lr"] * self.fn(self.last_epoch)

    def step(self) -> None:
        self.last_epoch += 1
        self._apply()

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch}

    def load_state_dict(self, sd: dict) -> None:
        self.last_epoch = sd["last_epoch"]
        self._apply()


def build_lr_scheduler(optimizer, config: TrainingConfig) -> LambdaLR:
    return LambdaLR(optimizer, lambda step: lr_factor(step, config))


def build_optimizer(model: nn.Module, config: TrainingConfig) -> AdamW:
    """Two groups: decayed, and not decayed when `ndim < 2` or the name contains bias / norm / embedding
    (so `embed_tokens` and `lm_head` are decayed, as in the reference)."""
    decay, no_decay = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (no_decay if is_no_decay(name, p) else decay).append(p)
    groups = [{"params": decay, "weight_decay": config.weight_decay}, {"params": no_decay, "weight_decay": 0.0}]
    return AdamW(groups, lr=config.learning_rate, betas=(config.beta1, config.beta2), eps=config.eps)


def count_parameters(model: nn.Module) -> dict[str, int]:
    total = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    return {"total": total, "trainable": trainable}


def get_grad_norm(model: nn.Module) -> float:
    """Global L2 norm of the gradients with a single host synchronisation."""
    sq = [(getattr(p, "main_grad", None) if getattr(p, "main_grad", None) is not None and getattr(p, "_grad_live", False)
           else p.grad) for p in model.parameters()]
    sq = [g.detach().float().pow(2).sum() for g in sq if g is not None]
    if not sq:
        return 0.0
    return float(torch.stack(sq).sum().sqrt().item())
