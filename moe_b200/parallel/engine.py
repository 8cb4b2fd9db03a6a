"""Training engine: flat parameter / gradient / optimiser-state buffers.

Replaces what the reference borrows from Accelerate + torch DDP + `torch.optim.AdamW`
(`train.py:398-403,507-509,546-556`, `src/utils/training.py:75-95`):

* every parameter is a view into one fp32 master buffer; on CUDA a bf16 compute copy and an fp32
  gradient accumulator of the same layout sit beside it.  Weight-gradient GEMM epilogues write
  into the accumulator directly, so there is no per-parameter `.grad` traffic;
* data parallelism is an all-reduce (average) over slices of the flat gradient buffer, issued
  per layer on a side stream while backward is still running;
* gradient norm, clipping and AdamW run over the flat buffers in a handful of launches with no
  host synchronisation; the same pass refreshes the bf16 copy.

On CPU the same class runs with plain torch ops (gloo for the all-reduce).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import oracle
from ..utils.profiling import phase

ALIGN = 64  # elements; keeps every slice 16-byte aligned in bf16 and 256-byte aligned in fp32


def is_no_decay(name: str, p: torch.Tensor) -> bool:
    """Weight-decay rule of the reference (`src/utils/training.py:79-84`)."""
    return p.ndim < 2 or "bias" in name or "norm" in name or "embedding" in name


@dataclass
class Slot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    decay: bool  # replicated and weight-decayed: the part that takes part in the overlapped reduce
    ep: bool = False  # expert-parallel shard: local to this rank, never all-reduced


class _LayerBoundary(torch.autograd.Function):
    """Identity in forward; in backward tells the engine that every gradient produced *after*
    this point of the forward pass is complete."""

    @staticmethod
    def forward(ctx, h, y, engine, tag):
        ctx.engine, ctx.tag = engine, tag
        return h.view_as(h), y.view_as(y)

    @staticmethod
    def backward(ctx, gh, gy):
        ctx.engine._on_boundary(ctx.tag)
        return gh, gy, None, None


class TrainEngine:
    HYPER_SLOTS = 8  # steps the host may stage ahead of the device
    sharded_params = False  # True in FsdpEngine: parameters exist only as per-rank slices

    def __init__(self, model: nn.Module, *, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0, process_group=None,
                 overlap_grad_reduce: bool = True, device: torch.device | str | None = None,
                 comm: str | None = None, shard_optimizer: bool = False):
        self.model = model
        self.lr, self.betas, self.eps = lr, betas, eps
        self.weight_decay, self.max_grad_norm = weight_decay, max_grad_norm
        self.group = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        self.step_count = 0
        if device is not None:
            model.to(device)
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not params:
            raise ValueError("model has no trainable parameters")
        self.device = params[0][1].device
        self.cuda = self.device.type == "cuda"
        self.overlap = overlap_grad_reduce and self.cuda and self.world > 1
        # ---- layout: decayed parameters first, then the rest; module order inside each part
        # regions: [replicated, decayed | expert-parallel shards (decayed) | not decayed]
        slots: list[Slot] = []
        off = 0
        for region in ("dense", "ep", "nodecay"):
            for n, p in params:
                is_ep = getattr(p, "_ep_shard", None) is not None
                nd = is_no_decay(n, p)
                kind = "nodecay" if nd else ("ep" if is_ep else "dense")
                if kind != region:
                    continue
                slots.append(Slot(n, p, off, p.numel(), kind == "dense", kind == "ep"))
                off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            if region == "dense":
                self.decay_end = off
            elif region == "ep":
                self.ep_end = off
        self.total = off
        self.has_ep = self.ep_end > self.decay_end
        if self.has_ep and not self.cuda:
            raise ValueError("expert-parallel parameters need CUDA (peer-memory kernels)")
        self.slots = slots
        self.by_name = {s.name: s for s in slots}
        dev = self.device
        # gradient reduction: "p2p" = own NVLink kernel over symmetric memory (fused average + norm
        # partials), "nccl" = library all-reduce.  Default: p2p on CUDA with up to 8 ranks.
        comm = comm or os.environ.get("MOE_B200_COMM") or ("p2p" if self.cuda and 1 < self.world <= 8 else "nccl")
        self.comm = comm if (self.cuda and self.world > 1) else "none"
        self.p32 = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self._peers = None
        self._fused_ar = None
        self._comm_stream = None
        if self.comm == "p2p":
            from .symm import PeerBuffers

            self._peers = PeerBuffers(self.total, dev, process_group)
            self.g32 = self._peers.grad
        else:
            self.g32 = torch.zeros(self.total, dtype=torch.float32, device=dev)
        # sharded optimizer (ZeRO stage 1 over the NVLink domain): each rank keeps Adam moments only for
        # the slice of every gradient bucket it reduces, updates that slice and stores the new bf16
        # weights into every rank's compute copy
        self.sharded = bool(shard_optimizer) and self.world > 1
        if self.sharded and self.comm != "p2p":
            raise ValueError("shard_optimizer needs the peer-memory gradient path (CUDA, comm='p2p', <= 8 ranks)")
        self._layer_offs = self.layer_offsets()
        self._plan_segments()
        self.m = torch.zeros(self._moment_numel, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self._moment_numel, dtype=torch.float32, device=dev)
        if self.sharded:
            self._peers.add_param_copy(self.total)
            self.p16 = self._peers.p16
        else:
            self.p16 = torch.zeros(self.total, dtype=torch.bfloat16, device=dev) if self.cuda else None
        for s in slots:
            view = self.p32[s.offset:s.offset + s.numel].view(s.param.shape)
            view.copy_(s.param.data)
            s.param.data = view
            gview = self.g32[s.offset:s.offset + s.numel].view(s.param.shape)
            if self.cuda:
                s.param._bf16 = self.p16[s.offset:s.offset + s.numel].view(s.param.shape)
                s.param.main_grad = gview
                s.param._grad_live = False
            else:
                s.param.grad = gview
        if self.cuda:
            self._norm_ss = torch.zeros(1, dtype=torch.float32, device=dev)
            self._coef = torch.ones(2, dtype=torch.float32, device=dev)
            # {lr, 1 - beta1^t, 1 - beta2^t}: read by the AdamW kernel from device memory, refreshed by
            # an async copy from pinned memory before each step (so a captured graph can be replayed)
            self._hyper = torch.zeros(3, dtype=torch.float32, device=dev)
            # The host runs ahead of the device, and an async copy reads pinned memory when it executes,
            # not when it is enqueued: every staged step gets its own pinned slot, and a slot is rewritten
            # only after the event recorded behind its copy has completed.
            self._hyper_ring = torch.zeros(self.HYPER_SLOTS, 3, dtype=torch.float32).pin_memory()
            self._hyper_events: list = [None] * self.HYPER_SLOTS
            self._hyper_next = 0
            self._coef_ep = torch.ones(1, dtype=torch.float32, device=dev)
            from ..ops import _ext

            self._ext = _ext.load()
            self._ss_scratch = torch.empty(self._ext.sumsq_blocks(self.total), dtype=torch.float32, device=dev)
            self._fuse_adjacent()
            self.refresh_compute_copy()
            self._comm_stream = torch.cuda.Stream(device=dev) if self.world > 1 else None
            if self._peers is not None:
                from ..ops import gemm as _G
                from .symm import FusedAllReduce

                pb = self._peers
                self._fused_ar = FusedAllReduce(self._ext, pb.grad_ptrs, pb.flag_ptrs, pb.norm_ptrs, pb.multicast_ptr,
                                                pb.rank, pb.world, dev, _G.status_word(dev))
        inner = getattr(self.model, "model", None)
        if inner is not None and hasattr(inner, "_boundary_fn"):
            inner._boundary_fn = self.boundary if self.overlap else None
        self.end_step_hooks: list = []
        self._grad_norm = None
        self._reduced_upto = self.total  # everything at or above this offset has been handed to the reducer
        self._pending = []
        self._boundaries: dict[int, int] = {}
        # True while a micro-batch other than the last one of the step runs: its gradients only
        # accumulate locally, the buckets are reduced during the last micro-batch's backward
        # (what `accelerator.accumulate` / DDP `no_sync` do in the reference, `train.py:546`)
        self.accumulating = False
        self._timeline = None  # list of (label, event) while a device timeline is being recorded

    # ------------------------------------------------------------------ set-up helpers
    def _fuse_adjacent(self) -> None:
        """Give attention / dense-MLP modules one matrix view over projections that sit side by side."""
        from ..models.backbone import Attention, DenseMLP

        def adjacent(ws):
            ss = [self._slot_of(w) for w in ws]
            if any(s is None for s in ss):
                return None
            for a, b in zip(ss, ss[1:]):
                if a.offset + a.numel != b.offset:
                    return None
            rows = sum(w.shape[0] for w in ws)
            cols = ws[0].shape[1]
            o = ss[0].offset
            return (self.p16[o:o + rows * cols].view(rows, cols), self.g32[o:o + rows * cols].view(rows, cols))

        for mod in self.model.modules():
            if isinstance(mod, Attention):
                mod._fused_qkv = adjacent([mod.q_proj.weight, mod.k_proj.weight, mod.v_proj.weight])
            elif isinstance(mod, DenseMLP):
                mod._fused_gate_up = adjacent([mod.gate_proj.weight, mod.up_proj.weight])

    def bucket_ranges(self) -> list[tuple[int, int]]:
        """The (lo, hi) slices of the replicated, decayed region in the order backward hands them to the
        reducer: one per decoder layer from the last to the first, then whatever lies below layer 0."""
        d = self.decay_end
        if d == 0:
            return []
        if not self.overlap:
            return [(0, d)]
        out, upto = [], d
        for off in reversed([o for o in self._layer_offs if o is not None]):
            if off < upto:
                out.append((off, upto))
                upto = off
        if upto > 0:
            out.append((0, upto))
        return out

    def owned_slice(self, lo: int, hi: int, rank: int | None = None) -> tuple[int, int]:
        """The part of bucket [lo, hi) that `rank` reduces and updates; same arithmetic as the reduce kernel
        (whole float4 groups, ceil-divided over the ranks)."""
        rank = self.rank if rank is None else rank
        n4 = (hi - lo) // 4
        per = (n4 + self.world - 1) // self.world
        a = min(per * rank, n4)
        b = min(a + per, n4)
        return lo + 4 * a, lo + 4 * b

    def _plan_segments(self) -> None:
        """Update segments (p_lo, p_hi, m_lo, weight_decay, kind); kind: 0 replicated, 1 expert shard,
        2 owned slice of a sharded bucket.  `m_lo` indexes the moment buffers."""
        self.rank = dist.get_rank(self.group) if self.world > 1 else 0
        d, pe, wd = self.decay_end, self.ep_end, self.weight_decay
        segs = []
        if not self.sharded:
            if d > 0:
                segs.append((0, d, 0, wd, 0))
            if pe > d:
                segs.append((d, pe, d, wd, 1))
            if self.total > pe:
                segs.append((pe, self.total, pe, 0.0, 0))
            self._moment_numel = self.total
        else:
            moff = 0
            for lo, hi in self.bucket_ranges():
                a, b = self.owned_slice(lo, hi)
                if b > a:
                    segs.append((a, b, moff, wd, 2))
                    moff += b - a
            if pe > d:
                segs.append((d, pe, moff, wd, 1))
                moff += pe - d
            if self.total > pe:
                segs.append((pe, self.total, moff, 0.0, 0))
                moff += self.total - pe
            self._moment_numel = moff
        self._segments = segs
        self._bucket_set = set(self.bucket_ranges())

    def _moment_index(self, kind_filter=None):
        return [(p_lo, p_hi, m_lo) for p_lo, p_hi, m_lo, _, k in self._segments if kind_filter is None or k in kind_filter]

    def _slot_of(self, p) -> Slot | None:
        for s in self.slots:
            if s.param is p:
                return s
        return None

    def refresh_compute_copy(self) -> None:
        if self.cuda:
            self._ext.cast_bf16(self.p32, self.p16)

    # ---------------------------------------------------------------- backward overlap
    def boundary(self, h: torch.Tensor, y: torch.Tensor, layer_idx: int):
        """Called by the decoder at the input of layer `layer_idx` with (residual stream, normed input).
        Backward reaches this node only after every gradient of layers >= layer_idx is complete."""
        if not self.overlap or self.accumulating or not (h.requires_grad and y.requires_grad):
            return h, y
        off = self._layer_offs[layer_idx]
        if off is None:
            return h, y
        return _LayerBoundary.apply(h, y, self, off)

    def layer_offsets(self) -> list[int]:
        """Lowest flat offset (within the decayed part) owned by each decoder layer, in layer order."""
        outs = []
        layers = getattr(getattr(self.model, "model", None), "layers", [])
        for i, _ in enumerate(layers):
            pre = f"model.layers.{i}."
            offs = [s.offset for s in self.slots if s.name.startswith(pre) and s.decay]
            outs.append(min(offs) if offs else None)
        return outs

    def _on_boundary(self, first_offset: int) -> None:
        # decayed region [first_offset, _reduced_upto) is final: reduce it now on the side stream
        hi = min(self._reduced_upto, self.decay_end)
        if first_offset < hi:
            self._launch_reduce(first_offset, hi)
            self._reduced_upto = first_offset

    # ---- device timeline of one step (CUDA events on the streams the work runs on; eager mode only)
    def start_timeline(self) -> None:
        self._timeline = []
        self.mark("step_start")

    def mark(self, label: str, stream=None) -> None:
        if self._timeline is None or not self.cuda:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream if stream is not None else torch.cuda.current_stream(self.device))
        self._timeline.append((label, ev))

    def timeline_report(self) -> list[tuple[str, float]]:
        """(label, milliseconds since `step_start`) for every mark, after synchronising the device."""
        tl, self._timeline = self._timeline or [], None
        if not tl:
            return []
        torch.cuda.synchronize(self.device)
        t0 = tl[0][1]
        return [(label, round(t0.elapsed_time(ev), 4)) for label, ev in tl]

    def _launch_reduce(self, lo: int, hi: int, final: bool = False) -> None:
        if self.world == 1 or hi <= lo:
            return
        self._zero_dead(lo, hi)
        if self.sharded and hi <= self.decay_end and (lo, hi) not in self._bucket_set:
            raise RuntimeError(f"gradient bucket [{lo}, {hi}) is not one of the planned optimizer shards")
        chunk = self.g32[lo:hi]
        if self.cuda and self._fused_ar is not None:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ev)
                self.mark(f"reduce[{lo}:{hi}]_start", self._comm_stream)
                with phase("comm"):
                    self._fused_ar.reduce(lo, hi - lo, final, publish=not (self.sharded and hi <= self.decay_end))
                self.mark(f"reduce[{lo}:{hi}]_end", self._comm_stream)
        elif self.cuda:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ev)
                work = dist.all_reduce(chunk, op=dist.ReduceOp.AVG, group=self.group, async_op=True)
            self._pending.append(work)
        else:
            dist.all_reduce(chunk, op=dist.ReduceOp.SUM, group=self.group)
            chunk.div_(self.world)

    def _zero_dead(self, lo: int, hi: int) -> None:
        """Parameters that received no gradient this step must contribute zeros."""
        if not self.cuda:
            return
        for s in self.slots:
            if lo <= s.offset < hi:
                if s.param.grad is not None:  # a gradient that came through ordinary autograd
                    if s.param._grad_live:
                        s.param.main_grad.add_(s.param.grad)
                    else:
                        s.param.main_grad.copy_(s.param.grad)
                    s.param.grad = None
                    s.param._grad_live = True
                if not s.param._grad_live:
                    s.param.main_grad.zero_()
                    s.param._grad_live = True

    # ------------------------------------------------------------------------- step
    def zero_grad(self) -> None:
        if self.cuda:
            for s in self.slots:
                s.param._grad_live = False
                s.param.grad = None
        else:
            self.g32.zero_()
            for s in self.slots:  # autograd may have replaced the view
                g = self.g32[s.offset:s.offset + s.numel].view(s.param.shape)
                if s.param.grad is None or s.param.grad.data_ptr() != g.data_ptr():
                    s.param.grad = g
        self._reduced_upto = self.total
        self._pending = []

    def reduce_gradients(self) -> None:
        """Finish the data-parallel average of whatever has not been reduced during backward."""
        if not self.cuda:
            for s in self.slots:
                g = self.g32[s.offset:s.offset + s.numel].view(s.param.shape)
                if s.param.grad is not None and s.param.grad.data_ptr() != g.data_ptr():
                    g.copy_(s.param.grad)
                    s.param.grad = g
        if self.world == 1:
            self._zero_dead(0, self.total)
            return
        # the undecayed tail (norm weights) and anything below the last boundary
        hi = min(self._reduced_upto, self.decay_end)
        tail = self.total > self.ep_end
        if self.has_ep:
            self._account_ep_norm()
        self._launch_reduce(0, hi, final=not tail)
        self._launch_reduce(self.ep_end, self.total, final=True)
        if self._fused_ar is not None and hi <= 0 and not tail:
            raise RuntimeError("no final gradient bucket was launched")
        self._reduced_upto = 0
        for w in self._pending:
            w.wait()
        self._pending = []
        if self.cuda and self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        if self.cuda and self._fused_ar is not None:
            self._fused_ar.end_step()
        for hook in self.end_step_hooks:
            hook()

    def set_hyper(self, lr: float | None = None) -> None:
        """Stage the learning rate and Adam bias corrections of the NEXT step on the device."""
        if lr is not None:
            self.lr = lr
        if self.cuda:
            t = self.step_count + 1
            i = self._hyper_next
            self._hyper_next = (i + 1) % self.HYPER_SLOTS
            ev = self._hyper_events[i]
            if ev is not None:
                ev.synchronize()  # the copy that read this slot has run
            slot = self._hyper_ring[i]
            slot[0] = self.lr
            slot[1] = 1.0 - self.betas[0] ** t
            slot[2] = 1.0 - self.betas[1] ** t
            self._hyper.copy_(slot, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._hyper_events[i] = ev

    def _account_ep_norm(self) -> None:
        """Expert shards are not reduced: every token of every rank already contributed to the owner's
        gradient.  What remains is the 1/world of the data-parallel mean (applied inside AdamW) and this
        rank's share of the global gradient norm, added to the running sum the fused all-reduce keeps."""
        self._zero_dead(self.decay_end, self.ep_end)
        e = self._ext
        e.sumsq(self.g32[self.decay_end:self.ep_end], self._ss_scratch, self._norm_ss, False)
        if self._fused_ar is None:
            raise RuntimeError("expert parallelism requires the peer-memory gradient path (comm='p2p')")
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ev)
            self._fused_ar.state_f[1:2].add_(self._norm_ss / float(self.world * self.world))

    def step(self, lr: float | None = None, *, update_hyper: bool = True, count: bool = True) -> torch.Tensor:
        """Reduce, clip by global norm, AdamW.  Returns the (pre-clip) gradient norm as a tensor.
        `update_hyper=False, count=False` is for CUDA-graph capture: the caller stages the
        hyper-parameters and advances the step counter around each replay."""
        if update_hyper:
            self.set_hyper(lr)
        elif lr is not None:
            self.lr = lr
        self.mark("backward_end")
        with phase("comm"):
            self.reduce_gradients()
        self.mark("reduces_joined")
        if count:
            self.step_count += 1
        b1, b2 = self.betas
        if self.cuda:
            e = self._ext
            if self._fused_ar is not None:  # the reduce kernels already produced every rank's sum of squares
                e.clip_coef_multi(self._peers.norm, self.world, float(self.max_grad_norm or 0.0), self._coef)
            else:
                e.sumsq(self.g32, self._ss_scratch, self._norm_ss, False)
                e.clip_coef(self._norm_ss, float(self.max_grad_norm or 0.0), self._coef)
            if self.ep_end > self.decay_end:  # expert shards: clip coefficient times the 1/world of the mean
                torch.div(self._coef[:1], float(self.world), out=self._coef_ep)
            for p_lo, p_hi, m_lo, wd, kind in self._segments:
                n = p_hi - p_lo
                e.adamw(self.p32[p_lo:p_hi], self.g32[p_lo:p_hi], self.m[m_lo:m_lo + n], self.v[m_lo:m_lo + n],
                        None if kind == 2 else self.p16[p_lo:p_hi], self._hyper, b1, b2, self.eps, wd,
                        self._coef_ep if kind == 1 else self._coef,
                        [q + 2 * p_lo for q in self._peers.p16_ptrs] if kind == 2 else [],
                        (self._peers.p16_mc + 2 * p_lo) if kind == 2 and self._peers.p16_mc else 0)
            self.mark("adamw_end")
            if self.sharded:  # every rank's stores into this rank's bf16 copy have landed after this
                self._fused_ar.param_barrier()
                self.mark("param_barrier_end")
            self._grad_norm = self._coef[1]
            if self._peers is not None and getattr(self._peers, "_guard", 0):
                self._peers.check_canaries()
        else:
            norm = self.g32.norm()
            coef = 1.0
            if self.max_grad_norm and self.max_grad_norm > 0:
                coef = float(min(1.0, self.max_grad_norm / (norm.item() + 1e-6)))
            d = self.decay_end
            for lo, hi, wd in ((0, d, self.weight_decay), (self.ep_end, self.total, 0.0)):
                if hi > lo:
                    oracle.adamw_step_(self.p32[lo:hi], self.g32[lo:hi], self.m[lo:hi], self.v[lo:hi], lr=self.lr,
                                       beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd, step=self.step_count,
                                       grad_scale=coef)
            self._grad_norm = norm
        return self._grad_norm

    # ------------------------------------------------------------------------ state
    def grad_norm(self) -> torch.Tensor | None:
        return self._grad_norm

    def full_moments(self) -> tuple[torch.Tensor, torch.Tensor]:
        """Adam moments in parameter layout.  Collective when the optimizer is sharded: every rank fills in
        what it owns and a sum over ranks assembles the rest."""
        if not self.sharded:
            return self.m, self.v
        outs = []
        for src in (self.m, self.v):
            full = torch.zeros(self.total, dtype=torch.float32, device=self.device)
            for p_lo, p_hi, m_lo, _, kind in self._segments:
                if kind == 2 or self.rank == 0 or kind == 1:  # replicated tails: taken from rank 0 only
                    full[p_lo:p_hi].copy_(src[m_lo:m_lo + p_hi - p_lo])
            d, pe = self.decay_end, self.ep_end
            if d > 0:
                dist.all_reduce(full[:d], group=self.group)
            if self.total > pe:
                dist.all_reduce(full[pe:], group=self.group)
            outs.append(full)
        return outs[0], outs[1]

    def sync_master(self) -> None:
        """Sharded optimizer: bring the fp32 master weights of every rank up to date (each rank only
        advances the slices it owns).  Collective; call before reading `state_dict()`."""
        if not self.sharded or self.decay_end == 0:
            return
        own = torch.zeros(self.decay_end, dtype=torch.float32, device=self.device)
        for p_lo, p_hi, _, _, kind in self._segments:
            if kind == 2:
                own[p_lo:p_hi].copy_(self.p32[p_lo:p_hi])
        dist.all_reduce(own, group=self.group)
        # float4 remainders of a bucket belong to nobody and never change
        mask = torch.zeros(self.decay_end, dtype=torch.bool, device=self.device)
        for lo, hi in self.bucket_ranges():
            mask[lo:lo + (hi - lo) // 4 * 4] = True
        self.p32[:self.decay_end] = torch.where(mask, own, self.p32[:self.decay_end])

    # ---- sharded checkpoints: which flat ranges this rank writes, and which it must read back
    def export_state_ranges(self) -> list[tuple[str, int, int, torch.Tensor]]:
        """(kind, flat_lo, flat_hi, tensor) with kind 'p' (fp32 master), 'm', 'v': every element of the training
        state is named by exactly one rank (replicated parts by rank 0, sharded parts by their owner)."""
        out = []
        rank0 = self.rank == 0 if hasattr(self, "rank") else True
        for p_lo, p_hi, m_lo, _, kind in self._segments:
            n = p_hi - p_lo
            if kind == 0 and not rank0:
                continue
            out.append(("p", p_lo, p_hi, self.p32[p_lo:p_hi]))
            out.append(("m", p_lo, p_hi, self.m[m_lo:m_lo + n]))
            out.append(("v", p_lo, p_hi, self.v[m_lo:m_lo + n]))
        return out

    def import_state_ranges(self) -> list[tuple[str, int, int, torch.Tensor]]:
        """Destinations this rank fills when loading: all master values it holds, its part of the moments."""
        out = [("p", 0, self.total, self.p32)]
        for p_lo, p_hi, m_lo, _, _ in self._segments:
            n = p_hi - p_lo
            out.append(("m", p_lo, p_hi, self.m[m_lo:m_lo + n]))
            out.append(("v", p_lo, p_hi, self.v[m_lo:m_lo + n]))
        return out

    def after_state_import(self) -> None:
        self.refresh_compute_copy()

    def optimizer_state_dict(self) -> dict:
        st = {"step": self.step_count, "lr": self.lr, "state": {}}
        m, v = self.full_moments()
        for s in self.slots:
            sl = slice(s.offset, s.offset + s.numel)
            st["state"][s.name] = {"exp_avg": m[sl].view(s.param.shape).detach().cpu().clone(),
                                   "exp_avg_sq": v[sl].view(s.param.shape).detach().cpu().clone()}
        return st

    def load_optimizer_state_dict(self, st: dict) -> None:
        self.step_count = int(st["step"])
        self.lr = float(st.get("lr", self.lr))
        if self.sharded:
            m = torch.zeros(self.total, dtype=torch.float32, device=self.device)
            v = torch.zeros_like(m)
        else:
            m, v = self.m, self.v
        for name, d in st["state"].items():
            s = self.by_name.get(name)
            if s is None:
                continue
            sl = slice(s.offset, s.offset + s.numel)
            m[sl].copy_(d["exp_avg"].reshape(-1))
            v[sl].copy_(d["exp_avg_sq"].reshape(-1))
        if self.sharded:
            for p_lo, p_hi, m_lo, _, _ in self._segments:
                self.m[m_lo:m_lo + p_hi - p_lo].copy_(m[p_lo:p_hi])
                self.v[m_lo:m_lo + p_hi - p_lo].copy_(v[p_lo:p_hi])

    def model_state_dict(self) -> dict:
        """Name -> tensor with the fp32 master values (call `sync_master()` first when the optimizer is sharded)."""
        return self.model.state_dict()

    def full_master(self) -> torch.Tensor:
        """The flat fp32 master buffer in parameter layout."""
        self.sync_master()
        return self.p32

    def load_model_state_dict(self, sd: dict, strict: bool = True) -> None:
        self.model.load_state_dict(sd, strict=strict)
        self.refresh_compute_copy()

    def broadcast_parameters(self, src: int = 0) -> None:
        """Make rank `src` authoritative (the reference gets this from DDP's initial broadcast)."""
        if self.world > 1:
            # expert-parallel shards [decay_end, ep_end) differ per rank by construction and stay untouched
            for lo, hi in ((0, self.decay_end), (self.ep_end, self.total)):
                if hi > lo:
                    dist.broadcast(self.p32[lo:hi], src=src, group=self.group)
            for mod in self.model.modules():
                for b in mod.buffers(recurse=False):
                    dist.broadcast(b, src=src, group=self.group)
            self.refresh_compute_copy()
