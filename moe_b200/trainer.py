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

from .ops import _ext
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
    router_stats: object | None = None  # kernel path: per-layer routing statistics of the last micro-batch


class Trainer:
    def __init__(self, model, cfg: TrainingConfig, *, device=None, process_group=None, is_moe: bool = True,
                 overlap_grad_reduce: bool = True, cuda_graph: bool = False, graph_warmup_steps: int = 2,
                 ep_capacity_factor: float = 2.0, comm: str | None = None, shard_optimizer: bool = False,
                 shard_params: bool = False):
        self.model = model
        self.cfg = cfg
        self.is_moe = is_moe
        if shard_params:  # ZeRO-3: parameters, gradients and optimizer state sharded, pulled per layer
            from .parallel.fsdp import FsdpEngine

            self.engine = FsdpEngine(model, lr=cfg.learning_rate, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps,
                                     weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                     process_group=process_group, device=device)
        else:
            self.engine = TrainEngine(model, lr=cfg.learning_rate, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps,
                                      weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                      process_group=process_group, device=device,
                                      overlap_grad_reduce=overlap_grad_reduce, comm=comm,
                                      shard_optimizer=shard_optimizer)
        self.device = self.engine.device
        # expert parallelism: parameters that are shards of an expert bank get the peer-memory context
        self.ep = None
        if self.engine.has_ep:
            from .parallel.ep import EPContext

            self.ep = EPContext(model.config.num_experts, process_group, self.device, ep_capacity_factor)
            for s in self.engine.slots:
                if s.ep:
                    s.param._ep = self.ep
            self.engine.end_step_hooks.append(self.ep.end_step)
        self.global_step = 0
        self.world = self.engine.world
        # whole-step CUDA graph: the step is captured once (after a few eager steps have run every
        # lazy initialisation) and replayed with new inputs / learning rate, which removes the
        # per-op launch and autograd overhead of several hundred small launches per step
        self.use_graph = bool(cuda_graph) and self.device.type == "cuda"
        self._graph = None
        self._graph_key = None
        self._graph_warmup = graph_warmup_steps
        self._capture_stream = None
        self._eager_steps = 0
        if cfg.gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
            model.gradient_checkpointing_enable()
            if self.ep is not None:
                self.ep.share_buffers = True
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
        if self.use_graph and self._eager_steps >= self._graph_warmup:
            return self._graph_step(micro_batches)
        self._eager_steps += 1
        lr = self.current_lr()
        out, tokens = self._forward_backward([{k: self._to_device(v) for k, v in mb.items()} for mb in micro_batches])
        gn = self.engine.step(lr)
        self.global_step += 1
        return self._result(out, gn, lr, tokens)

    def _forward_backward(self, dev_batches):
        n = len(dev_batches)
        self.engine.zero_grad()
        if self.ep is not None:
            self.ep.begin_step()
        scale = 1.0 / n
        out, tokens = None, 0
        for i, mb in enumerate(dev_batches):
            ids, labels = mb["input_ids"], mb["labels"]
            tokens += ids.numel()
            kw = {"output_router_logits": True} if self.is_moe else {}
            # bucket reduces are launched from the backward of the last micro-batch only
            self.engine.accumulating = i < n - 1
            try:
                out = self.model(input_ids=ids, labels=labels, loss_scale=scale, **kw)
                loss = out.loss * scale if n > 1 else out.loss
                loss.backward()
            finally:
                self.engine.accumulating = False
        return out, tokens

    def _result(self, out, gn, lr, tokens) -> StepResult:
        return StepResult(loss=out.loss.detach(), ce_loss=_d(out.ce_loss), aux_loss=_d(out.aux_loss),
                          seq_aux_loss=_d(out.seq_aux_loss), grad_norm=gn, lr=lr,
                          router_logits=None if out.router_logits is None else tuple(t.detach() for t in out.router_logits),
                          tokens=tokens * self.world, router_stats=getattr(out, "router_stats", None))

    def _graph_step(self, micro_batches) -> StepResult:
        key = tuple((tuple(mb["input_ids"].shape), tuple(mb["labels"].shape)) for mb in micro_batches)
        if self._graph is None or key != self._graph_key:
            self._capture(micro_batches, key)
        for st, mb in zip(self._static_in, micro_batches):
            st["input_ids"].copy_(mb["input_ids"], non_blocking=True)
            st["labels"].copy_(mb["labels"], non_blocking=True)
        lr = self.current_lr()
        self.engine.set_hyper(lr)
        self._graph.replay()
        _ext.add_launches(self._graph_launches)
        self.engine.step_count += 1
        self.global_step += 1
        out, gn, tokens = self._static_out
        return self._result(out, gn, lr, tokens)

    def _capture(self, micro_batches, key) -> None:
        self._graph = None
        self._static_in = [{"input_ids": torch.empty_like(mb["input_ids"], device=self.device),
                            "labels": torch.empty_like(mb["labels"], device=self.device)} for mb in micro_batches]
        for st, mb in zip(self._static_in, micro_batches):  # valid token ids while capturing
            st["input_ids"].copy_(mb["input_ids"])
            st["labels"].copy_(mb["labels"])
        # Libraries keep lazily created per-stream state (workspaces, handles); creating it inside a
        # capture invalidates the capture.  So run one forward/backward on the capture stream first.
        # That dry run must leave no trace: gradients are reset by the step's own zero_grad, router
        # token counters are put back.
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        cs = self._capture_stream
        counters = [b for n, b in self.model.named_buffers() if n.endswith("local_tokens_per_expert")]
        saved = [c.clone() for c in counters]
        cs.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(cs):
            self._forward_backward(self._static_in)
            # close the dry run's gradient phase as a step would (no update): the bucket reduces it launched
            # have added to the running squared norm and taken flag epochs, which the final reduce settles
            self.engine.reduce_gradients()
            for c, sv in zip(counters, saved):
                c.copy_(sv)
        torch.cuda.current_stream(self.device).wait_stream(cs)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        l0 = _ext.launch_count()
        # thread-local capture mode: NCCL's watchdog thread may touch CUDA while this thread captures
        # no garbage collection while capturing: a collection could free tensors of earlier eager
        # steps in the middle of the capture, and the allocator's bookkeeping for blocks that were
        # used on other streams is not capturable
        import gc

        gc_was_on = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            with torch.cuda.graph(g, stream=cs, capture_error_mode="thread_local"):
                out, tokens = self._forward_backward(self._static_in)
                gn = self.engine.step(update_hyper=False, count=False)
        finally:
            if gc_was_on:
                gc.enable()
        self._graph, self._graph_key = g, key
        self._graph_launches = _ext.launch_count() - l0  # kernels of ours inside one replay
        _ext.add_launches(-self._graph_launches)  # capture itself ran nothing
        self._static_out = (out, gn, tokens)


def _d(t):
    return t.detach() if isinstance(t, torch.Tensor) else t
