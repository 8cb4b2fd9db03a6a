"""`Trainer`: the public training-step API (what `train.py` and `bench.py` call).

One optimizer step = `gradient_accumulation` micro-batches through the model, backward, gradient
average over data-parallel ranks (overlapped with backward), global-norm clip, AdamW, LR schedule
(`train.py:546-572` of the reference, without Accelerate).  Micro-batches arrive as host tensors
(pinned when possible) and are copied to the device here, so a caller that times `train_step`
times the host-to-device input copy too.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .parallel.engine import TrainEngine
from .utils.training import TrainingConfig, lr_factor


@dataclass
class StepResult:
    loss: torch.Tensor            # last micro-batch, device scalar (total loss)
    ce_loss: torch.Tensor | None
    aux_loss: torch.Tensor | None
    seq_aux_loss: torch.Tensor | None
    grad_norm: torch.Tensor
    lr: float
    router_logits: tuple | None = None
    tokens: int = 0


class Trainer:
    def __init__(self, model, cfg: TrainingConfig, *, device=None, process_group=None, is_moe: bool = True,
                 overlap_grad_reduce: bool = True):
        self.model = model
        self.cfg = cfg
        self.is_moe = is_moe
        self.engine = TrainEngine(model, lr=cfg.learning_rate, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps,
                                  weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                  process_group=process_group, device=device,
                                  overlap_grad_reduce=overlap_grad_reduce)
        self.device = self.engine.device
        self.global_step = 0
        self.world = self.engine.world
        if cfg.gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
            model.gradient_checkpointing_enable()
        model.train()

    # LR for the optimizer step about to be taken (scheduler semantics of LambdaLR: step k uses factor(k))
    def current_lr(self) -> float:
        return self.cfg.learning_rate * lr_factor(self.global_step, self.cfg)

    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device:
            return t
        return t.to(self.device, non_blocking=True)

    def train_step(self, micro_batches) -> StepResult:
        """`micro_batches`: one dict or a list of dicts with `input_ids` and `labels` `[B, S]` (int64)."""
        if isinstance(micro_batches, dict):
            micro_batches = [micro_batches]
        n = len(micro_batches)
        eng = self.engine
        eng.zero_grad()
        scale = 1.0 / n
        out = None
        tokens = 0
        for mb in micro_batches:
            ids = self._to_device(mb["input_ids"])
            labels = self._to_device(mb["labels"])
            tokens += ids.numel()
            kw = {"output_router_logits": True} if self.is_moe else {}
            out = self.model(input_ids=ids, labels=labels, loss_scale=scale, **kw)
            loss = out.loss * scale if n > 1 else out.loss
            loss.backward()
        lr = self.current_lr()
        gn = eng.step(lr)
        self.global_step += 1
        return StepResult(loss=out.loss.detach(), ce_loss=_d(out.ce_loss), aux_loss=_d(out.aux_loss),
                          seq_aux_loss=_d(out.seq_aux_loss), grad_norm=gn, lr=lr, router_logits=out.router_logits,
                          tokens=tokens * self.world)


def _d(t):
    return t.detach() if isinstance(t, torch.Tensor) else t
