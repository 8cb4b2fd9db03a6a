"""Fully sharded data parallelism (ZeRO stage 3) over one NVLink domain.

What the reference only has as an unused Accelerate recipe (`accelerate_configs/fsdp_8gpu.yaml:4-14`:
FULL_SHARD, BACKWARD_PRE prefetch, SHARDED_STATE_DICT), built on the peer-memory kernels of this package:

* The replicated, weight-decayed parameters are cut into *units*: the root unit (everything in front of
  decoder layer 0: the embedding and, in the global layout, the one expert bank every layer uses), one unit
  per decoder layer, and a head unit (`lm_head` when it is not tied).  Of every unit each rank owns one
  contiguous slice: the fp32 master values, both Adam moments, the reduced gradient and the bf16 compute
  copy of that slice are the only persistent per-parameter state a rank holds.
* Before a unit is used, its bf16 slices are pulled from all ranks' shard buffers (symmetric memory, plain
  peer loads issued by `allgather_bf16_kernel`) into a LOCAL staging buffer: the root unit into a buffer of
  its own once per step, layers and head into a ring of two slots.  The pull of unit u+1 runs on a side
  stream under the compute of unit u, forward and backward (backward-pre prefetch); the GEMMs' TMA only
  ever reads the local staging buffers.
* Gradients of a unit are written by the weight-gradient GEMM epilogues into a two-slot fp32 staging ring
  (symmetric memory); when the unit's backward is complete the reduce kernel runs in reduce-scatter form
  (fused 1/world and squared-norm partial) and the owned slice is added to the rank's gradient shard.  The
  root unit's gradient accumulates over all layers (global expert bank) and is reduce-scattered once.
* AdamW runs over the shard in one launch and writes the new bf16 slice; a flag barrier orders it before the
  next step's pulls.  Norm weights (the undecayed tail) stay replicated and are all-reduced; expert-parallel
  shards stay local, as in the other modes.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .engine import ALIGN, Slot, TrainEngine, is_no_decay


class _Unit:
    def __init__(self, name: str, lo: int, hi: int):
        self.name, self.lo, self.hi = name, lo, hi
        self.n = hi - lo
        self.per = 0      # elements of the unit every rank owns (uniform; the last rank's tail may be padding)
        self.soff = 0     # offset of the unit's piece inside every rank's shard buffers
        self.p_off = 0    # offset of the unit's staging area in the local bf16 buffer
        self.g_off = 0    # offset of the unit's staging area in the symmetric fp32 gradient buffer
        self.slots: list[Slot] = []
        self.gather_ev = None
        self.reduce_ev = None


class _FsdpBoundary(torch.autograd.Function):
    """Identity in forward.  In backward it runs when every gradient of unit `idx` is complete."""

    @staticmethod
    def forward(ctx, h, y, engine, idx):
        ctx.engine, ctx.idx = engine, idx
        return h.view_as(h), y.view_as(y)

    @staticmethod
    def backward(ctx, gh, gy):
        ctx.engine._unit_backward_done(ctx.idx)
        return gh, gy, None, None


class FsdpEngine(TrainEngine):
    """Same public surface as `TrainEngine` (zero_grad / step / grad_norm / state dicts), parameters,
    gradients and optimizer state sharded over the ranks."""

    sharded_params = True

    def __init__(self, model: nn.Module, *, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0, process_group=None,
                 device: torch.device | str | None = None):
        from ..ops import _ext
        from ..ops import gemm as _G
        from .symm import FusedAllReduce, PeerBuffers

        self.model = model
        self.lr, self.betas, self.eps = lr, betas, eps
        self.weight_decay, self.max_grad_norm = weight_decay, max_grad_norm
        self.group = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        if self.world not in (1, 2, 4, 8):
            raise ValueError("parameter sharding supports 1, 2, 4 or 8 ranks (one NVLink domain)")
        self.step_count = 0
        if device is not None:
            model.to(device)
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.device = params[0][1].device
        if self.device.type != "cuda":
            raise ValueError("parameter sharding needs CUDA (peer-memory kernels)")
        self.cuda, self.overlap, self.sharded, self.comm = True, True, True, "p2p"
        dev = self.device
        # ---- flat layout, identical to TrainEngine: [replicated decayed | expert-parallel | undecayed]
        slots: list[Slot] = []
        off = 0
        for region in ("dense", "ep", "nodecay"):
            for n, p in params:
                is_ep = getattr(p, "_ep_shard", None) is not None
                kind = "nodecay" if is_no_decay(n, p) else ("ep" if is_ep else "dense")
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
        self.slots = slots
        self.by_name = {s.name: s for s in slots}
        self._layer_offs = self.layer_offsets()
        # ---- units
        d = self.decay_end
        layer_lo = [o for o in self._layer_offs if o is not None]
        if len(layer_lo) != len(self._layer_offs) or sorted(layer_lo) != layer_lo:
            raise ValueError("every decoder layer must own replicated parameters, in module order")
        head = self.by_name.get("lm_head.weight")
        head_lo = head.offset if (head is not None and head.decay and layer_lo and head.offset >= layer_lo[-1]) else d
        cuts = layer_lo + [head_lo]
        self.root = _Unit("root", 0, layer_lo[0] if layer_lo else d)
        self.ring_units = [_Unit(f"layer{i}", cuts[i], cuts[i + 1]) for i in range(len(layer_lo))]
        if head_lo < d:
            self.ring_units.append(_Unit("head", head_lo, d))
        self.n_layers = len(layer_lo)
        units = [self.root] + self.ring_units
        soff = 0
        for u in units:
            n4 = u.n // 4
            u.per = (n4 + self.world - 1) // self.world * 4
            if u.per % 8 != 0:
                raise ValueError("unit size does not split into 16-byte bf16 pieces")
            u.soff = soff
            soff += u.per
            u.slots = [s for s in slots if s.decay and u.lo <= s.offset < u.hi]
        self.shard_total = soff
        max_ring = max([u.n for u in self.ring_units], default=0)
        # ---- local staging (bf16): [root | slot 0 | slot 1 | expert-parallel | undecayed tail]
        self._p_root, self._p_slot = 0, [self.root.n, self.root.n + max_ring]
        self._p_ep = self.root.n + 2 * max_ring
        self._p_tail = self._p_ep + (self.ep_end - self.decay_end)
        n_stage = self._p_tail + (self.total - self.ep_end)
        self.p16 = torch.zeros(n_stage, dtype=torch.bfloat16, device=dev)
        self._peers = PeerBuffers(n_stage, dev, process_group) if self.world > 1 else None
        self.g32 = self._peers.grad if self._peers is not None else torch.zeros(n_stage, dtype=torch.float32, device=dev)
        self.root.p_off = self.root.g_off = 0
        for i, u in enumerate(self.ring_units):
            u.p_off = u.g_off = self._p_slot[i % 2]
        # ---- persistent sharded state
        n_loc = self.total - self.decay_end  # expert-parallel shards + undecayed tail stay whole
        self.p32 = torch.zeros(self.shard_total + n_loc, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.p32)
        self.v = torch.zeros_like(self.p32)
        self.gshard = torch.zeros(self.shard_total, dtype=torch.float32, device=dev)
        if self._peers is not None:
            import torch.distributed._symmetric_memory as sm

            self.p16_shard = sm.empty(self.shard_total, dtype=torch.bfloat16, device=dev)
            self.p16_shard.zero_()
            torch.cuda.synchronize(dev)
            self._shard_handle = sm.rendezvous(self.p16_shard, self._peers.group)
            self._shard_ptrs = [int(p) for p in self._shard_handle.buffer_ptrs]
            dist.barrier(self._peers.group)
        else:
            self.p16_shard = torch.zeros(self.shard_total, dtype=torch.bfloat16, device=dev)
            self._shard_ptrs = [self.p16_shard.data_ptr()]
        self._ext = _ext.load()
        self._install_parameters(units)
        # ---- optimizer plumbing shared with TrainEngine
        self._norm_ss = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(2, dtype=torch.float32, device=dev)
        self._hyper = torch.zeros(3, dtype=torch.float32, device=dev)
        self._hyper_ring = torch.zeros(self.HYPER_SLOTS, 3, dtype=torch.float32).pin_memory()
        self._hyper_events = [None] * self.HYPER_SLOTS
        self._hyper_next = 0
        self._coef_ep = torch.ones(1, dtype=torch.float32, device=dev)
        self._ss_scratch = torch.empty(self._ext.sumsq_blocks(max(self.p32.numel(), 1)), dtype=torch.float32, device=dev)
        self._ss_scratch_comm = torch.empty_like(self._ss_scratch)  # for sums taken on the communication stream
        self._fused_ar = None
        self._comm_stream = torch.cuda.Stream(device=dev)
        self._gather_stream = torch.cuda.Stream(device=dev)
        if self._peers is not None:
            pb = self._peers
            self._fused_ar = FusedAllReduce(self._ext, pb.grad_ptrs, pb.flag_ptrs, pb.norm_ptrs, pb.multicast_ptr,
                                            pb.rank, pb.world, dev, _G.status_word(dev))
        self._fuse_adjacent()
        inner = getattr(self.model, "model", None)
        if inner is not None and hasattr(inner, "_boundary_fn"):
            inner._boundary_fn = self.boundary
            inner._boundary_after_last = True
        self.end_step_hooks: list = []
        self._grad_norm = None
        self._pending = []
        self.accumulating = False
        self._accum_step = False  # this step has reduced a layer unit for more than one micro-batch
        self._micro = 0            # micro-batches reduced into the gradient shard so far this step
        self._root_ready = False   # root unit gathered for the current parameter version
        self._in_backward_of = None
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ set-up helpers
    def _stage_off(self, s: Slot) -> int:
        """Offset of a parameter inside the staging buffers (bf16 copy and fp32 gradient share it)."""
        if s.decay:
            for u in [self.root] + self.ring_units:
                if u.lo <= s.offset < u.hi:
                    return u.p_off + (s.offset - u.lo)
            raise RuntimeError(f"parameter {s.name} belongs to no unit")
        if s.ep:
            return self._p_ep + (s.offset - self.decay_end)
        return self._p_tail + (s.offset - self.ep_end)

    def _local_off(self, s: Slot) -> int:
        """Offset of an expert-parallel / undecayed parameter in the fp32 state buffers (after the shard)."""
        return self.shard_total + (s.offset - self.decay_end)

    def _install_parameters(self, units) -> None:
        """Move the freshly initialised full parameters into the shards and point the modules at the staging
        buffers.  Sharded parameters keep no full fp32 tensor: `.data` becomes a zero-stride placeholder of
        the right shape (shape and device are all the model code reads from it)."""
        r = self.rank
        placeholder = torch.zeros(1, dtype=torch.float32, device=self.device)
        for u in units:
            own_lo = u.lo + u.per * r
            own_hi = min(own_lo + u.per, u.hi)
            for s in u.slots:
                a, b = max(s.offset, own_lo), min(s.offset + s.numel, own_hi)
                if b > a:  # the part of this parameter that falls into the owned slice
                    src = s.param.data.reshape(-1)[a - s.offset:b - s.offset].float()
                    self.p32[u.soff + (a - own_lo):u.soff + (b - own_lo)].copy_(src)
        self._ext.cast_bf16(self.p32[:self.shard_total], self.p16_shard)
        for s in self.slots:
            so = self._stage_off(s)
            s.param._bf16 = self.p16[so:so + s.numel].view(s.param.shape)
            s.param.main_grad = self.g32[so:so + s.numel].view(s.param.shape)
            s.param._grad_live = False
            if s.decay:
                shape = tuple(s.param.shape)
                s.param.data = placeholder.expand(shape) if len(shape) else placeholder[0]
            else:
                lo = self._local_off(s)
                view = self.p32[lo:lo + s.numel].view(s.param.shape)
                view.copy_(s.param.data)
                s.param.data = view
                self._ext.cast_bf16(view.reshape(-1), s.param._bf16.reshape(-1))
        if self.world > 1:
            dist.barrier(self.group)

    def _fuse_adjacent(self) -> None:
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
            o = self._stage_off(ss[0])
            return (self.p16[o:o + rows * cols].view(rows, cols), self.g32[o:o + rows * cols].view(rows, cols))

        for mod in self.model.modules():
            if isinstance(mod, Attention):
                mod._fused_qkv = adjacent([mod.q_proj.weight, mod.k_proj.weight, mod.v_proj.weight])
            elif isinstance(mod, DenseMLP):
                mod._fused_gate_up = adjacent([mod.gate_proj.weight, mod.up_proj.weight])

    def refresh_compute_copy(self) -> None:
        self._ext.cast_bf16(self.p32[:self.shard_total], self.p16_shard)
        for s in self.slots:
            if not s.decay:
                self._ext.cast_bf16(s.param.data.reshape(-1), s.param._bf16.reshape(-1))
        self._root_ready = False

    def broadcast_parameters(self, src: int = 0) -> None:
        """Nothing to do: every rank builds the same seeded weights and keeps only its slices."""

    # ------------------------------------------------------------------ parameter pulls
    def _gather(self, u: _Unit, after_main: bool = True) -> None:
        """Pull unit `u` into its staging area on the gather stream; `u.gather_ev` marks completion."""
        main = torch.cuda.current_stream(self.device)
        gs = self._gather_stream
        if after_main:  # the staging area may still be read by kernels already enqueued on the main stream
            ev = torch.cuda.Event()
            ev.record(main)
            gs.wait_event(ev)
        with torch.cuda.stream(gs):
            self._ext.allgather_bf16([p + 2 * u.soff for p in self._shard_ptrs], u.per, u.n,
                                     self.p16[u.p_off:u.p_off + u.n], 64)
            u.gather_ev = torch.cuda.Event()
            u.gather_ev.record(gs)

    def _wait_unit(self, u: _Unit) -> None:
        if u.gather_ev is not None:
            torch.cuda.current_stream(self.device).wait_event(u.gather_ev)
            u.gather_ev = None

    def begin_step(self) -> None:
        """Start of a forward pass: the root unit (once per parameter version) and the first ring unit."""
        if not self._root_ready:
            self._gather(self.root)
            self._wait_unit(self.root)
            self._root_ready = True
        if self.ring_units:
            self._gather(self.ring_units[0])

    def boundary(self, h: torch.Tensor, y: torch.Tensor, idx: int):
        """Called by the decoder in front of ring unit `idx` (layer idx; idx = number of layers: the head)."""
        if idx >= len(self.ring_units):
            return h, y
        u = self.ring_units[idx]
        if u.gather_ev is None and idx == 0:
            self.begin_step()  # a forward pass that did not go through zero_grad (evaluation)
        self._wait_unit(u)
        if idx + 1 < len(self.ring_units):
            self._gather(self.ring_units[idx + 1])  # overwrites the slot of unit idx - 1, whose kernels are enqueued
        if torch.is_grad_enabled() and h.requires_grad and y.requires_grad:
            return _FsdpBoundary.apply(h, y, self, idx)
        return h, y

    # ------------------------------------------------------------------ backward
    def _unit_backward_done(self, idx: int) -> None:
        """Backward has passed the input of ring unit `idx`: its gradients are complete."""
        units = self.ring_units
        u = units[idx]
        # gradient slot of unit idx - 1 (written next) was last used by unit idx + 1: its reduce must be done
        if idx + 1 < len(units) and units[idx + 1].reduce_ev is not None:
            torch.cuda.current_stream(self.device).wait_event(units[idx + 1].reduce_ev)
            units[idx + 1].reduce_ev = None
        self._reduce_unit(u)
        # weights: unit idx - 1 runs next and must be resident; pull unit idx - 2 into the slot unit idx just freed
        if idx - 1 >= 0:
            self._wait_unit(units[idx - 1])
        if idx - 2 >= 0:
            self._gather(units[idx - 2])

    def _reduce_unit(self, u: _Unit, final: bool = False) -> None:
        """Reduce-scatter the unit's staged gradient and add the owned slice to the gradient shard."""
        self._zero_dead(u.lo, u.hi)
        main = torch.cuda.current_stream(self.device)
        cs = self._comm_stream
        ev = torch.cuda.Event()
        ev.record(main)
        own = self.g32[u.g_off + u.per * self.rank:u.g_off + u.per * self.rank + u.per]
        dst = self.gshard[u.soff:u.soff + u.per]
        valid = max(0, min(u.per, u.n - u.per * self.rank))
        with torch.cuda.stream(cs):
            cs.wait_event(ev)
            # With several micro-batches a layer unit is reduced once per micro-batch and the reduced slices are
            # added up in the gradient shard: the norm that clipping needs is that of the sum, so these reduces
            # do not count and `reduce_gradients` takes the squared norm of the accumulated shard instead.
            split = u is not self.root and (self.accumulating or self._accum_step)
            if split:
                self._accum_step = True
            if self._fused_ar is not None:
                self._fused_ar.reduce(u.g_off, u.n, final, publish=False, count_norm=not split)
            elif not split:
                self._ext.sumsq(self.g32[u.g_off:u.g_off + u.n], self._ss_scratch, self._norm_ss, True)
            if valid > 0:
                if self._micro == 0 or u is self.root:
                    dst[:valid].copy_(own[:valid])
                else:
                    dst[:valid].add_(own[:valid])
            u.reduce_ev = torch.cuda.Event()
            u.reduce_ev.record(cs)
        if u is not self.root:
            for s in u.slots:  # the slot is rewritten by another unit (or the next micro-batch)
                s.param._grad_live = False
        if self.ring_units and u is self.ring_units[0]:
            self._micro += 1  # the first ring unit is the last one a micro-batch's backward completes

    # ------------------------------------------------------------------------- step
    def zero_grad(self) -> None:
        for s in self.slots:
            s.param._grad_live = False
            s.param.grad = None
        self._micro = 0
        self._accum_step = False
        self._norm_ss.zero_()
        self._pending = []
        self.begin_step()

    def reduce_gradients(self) -> None:
        """End of backward: the root unit's reduce-scatter, the all-reduce of the undecayed tail."""
        main = torch.cuda.current_stream(self.device)
        for u in self.ring_units:  # a model run without boundaries in backward (no layers) has nothing here
            if u.reduce_ev is not None:
                main.wait_event(u.reduce_ev)
                u.reduce_ev = None
        tail = self.total > self.ep_end
        if self.has_ep:
            self._account_ep_norm_local()
        if self._accum_step:
            self._account_accumulated_units()
        self._reduce_unit(self.root, final=not tail and self._fused_ar is not None)
        if tail:
            self._zero_dead(self.ep_end, self.total)
            n = self.total - self.ep_end
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ev)
                if self._fused_ar is not None:
                    self._fused_ar.reduce(self._p_tail, n, True, publish=True)
                else:
                    self._ext.sumsq(self.g32[self._p_tail:self._p_tail + n], self._ss_scratch, self._norm_ss, True)
        main.wait_stream(self._comm_stream)
        main.wait_stream(self._gather_stream)
        self.root.reduce_ev = None
        if self._fused_ar is not None:
            self._fused_ar.end_step()
        for hook in self.end_step_hooks:
            hook()

    def _account_accumulated_units(self) -> None:
        """Squared norm of the layer units' accumulated (already averaged) gradient shards; on the communication
        stream, after the last unit's reduce-scatter and its add into the shard."""
        with torch.cuda.stream(self._comm_stream):
            ss = torch.zeros(1, dtype=torch.float32, device=self.device)
            for u in self.ring_units:
                valid = max(0, min(u.per, u.n - u.per * self.rank))
                if valid > 0:
                    self._ext.sumsq(self.gshard[u.soff:u.soff + valid], self._ss_scratch_comm, ss, True)
            if self._fused_ar is not None:
                self._fused_ar.state_f[1:2].add_(ss)
            else:
                self._norm_ss.add_(ss)

    def _account_ep_norm_local(self) -> None:
        """Expert-parallel shards are complete locally; their share of the squared norm joins the running sum."""
        self._zero_dead(self.decay_end, self.ep_end)
        n = self.ep_end - self.decay_end
        seg = self.g32[self._p_ep:self._p_ep + n]
        if self._fused_ar is None:
            self._ext.sumsq(seg, self._ss_scratch, self._norm_ss, True)
            return
        ss = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._ext.sumsq(seg, self._ss_scratch, ss, False)
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ev)
            self._fused_ar.state_f[1:2].add_(ss / float(self.world * self.world))

    def step(self, lr: float | None = None, *, update_hyper: bool = True, count: bool = True) -> torch.Tensor:
        if update_hyper:
            self.set_hyper(lr)
        elif lr is not None:
            self.lr = lr
        self.reduce_gradients()
        if count:
            self.step_count += 1
        b1, b2 = self.betas
        e = self._ext
        if self._fused_ar is not None:
            e.clip_coef_multi(self._peers.norm, self.world, float(self.max_grad_norm or 0.0), self._coef)
        else:
            e.clip_coef(self._norm_ss, float(self.max_grad_norm or 0.0), self._coef)
        st = self.shard_total
        if st > 0:  # the owned slices of every unit: one launch, new bf16 slice written next to them
            e.adamw(self.p32[:st], self.gshard, self.m[:st], self.v[:st], self.p16_shard, self._hyper, b1, b2, self.eps,
                    self.weight_decay, self._coef, [])
        if self.has_ep:
            torch.div(self._coef[:1], float(self.world), out=self._coef_ep)
            n = self.ep_end - self.decay_end
            lo = st
            e.adamw(self.p32[lo:lo + n], self.g32[self._p_ep:self._p_ep + n], self.m[lo:lo + n], self.v[lo:lo + n],
                    self.p16[self._p_ep:self._p_ep + n], self._hyper, b1, b2, self.eps, self.weight_decay,
                    self._coef_ep, [])
        if self.total > self.ep_end:
            n = self.total - self.ep_end
            lo = st + (self.ep_end - self.decay_end)
            e.adamw(self.p32[lo:lo + n], self.g32[self._p_tail:self._p_tail + n], self.m[lo:lo + n], self.v[lo:lo + n],
                    self.p16[self._p_tail:self._p_tail + n], self._hyper, b1, b2, self.eps, 0.0, self._coef, [])
        if self._fused_ar is not None:  # every rank's new slices are in place before anybody pulls them
            self._fused_ar.param_barrier()
            self._fused_ar.end_step()
        self._root_ready = False
        self._grad_norm = self._coef[1]
        return self._grad_norm

    # ------------------------------------------------------------------------ state
    def _gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        """Flat fp32 tensor in parameter layout `[0, total)` from every rank's `[shard | local]` buffer
        (collective; used by checkpoints and tests, not by the training step)."""
        full = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        st = self.shard_total
        if self.world > 1:
            parts = [torch.empty(st, dtype=torch.float32, device=self.device) for _ in range(self.world)]
            dist.all_gather(parts, shard[:st].contiguous(), group=self.group)
        else:
            parts = [shard[:st]]
        for u in [self.root] + self.ring_units:
            for r in range(self.world):
                a = u.lo + u.per * r
                b = min(a + u.per, u.hi)
                if b > a:
                    full[a:b].copy_(parts[r][u.soff:u.soff + (b - a)])
        full[self.decay_end:].copy_(shard[st:])
        return full

    def sync_master(self) -> None:
        """Nothing to bring up to date: masters exist only as shards (see `full_master`)."""

    def full_master(self) -> torch.Tensor:
        return self._gather_full(self.p32)

    def full_moments(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self._gather_full(self.m), self._gather_full(self.v)

    def model_state_dict(self) -> dict:
        """Parameter name -> full fp32 tensor (collective), plus the model's buffers."""
        full = self.full_master()
        sd = {}
        for s in self.slots:
            sd[s.name] = full[s.offset:s.offset + s.numel].view(s.param.shape).clone()
        own = dict(self.model.named_parameters())
        for k, v in self.model.state_dict().items():
            if k not in own and k not in sd:
                sd[k] = v
            elif k in own and k not in sd:  # a second name of a shared tensor (tied lm_head)
                for s in self.slots:
                    if s.param is own[k]:
                        sd[k] = sd[s.name]
        return sd

    def _scatter_full(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        r = self.rank
        for u in [self.root] + self.ring_units:
            a = u.lo + u.per * r
            b = min(a + u.per, u.hi)
            if b > a:
                shard[u.soff:u.soff + (b - a)].copy_(full[a:b])
        shard[self.shard_total:].copy_(full[self.decay_end:])

    def load_model_state_dict(self, sd: dict, strict: bool = True) -> None:
        full = self.full_master()
        for s in self.slots:
            if s.name in sd:
                full[s.offset:s.offset + s.numel].copy_(sd[s.name].reshape(-1).to(full))
            elif strict:
                raise KeyError(f"missing parameter {s.name}")
        self._scatter_full(full, self.p32)
        bufs = {k: v for k, v in sd.items() if k not in self.by_name}
        own = dict(self.model.named_buffers())
        for k, v in bufs.items():
            if k in own:
                own[k].copy_(v)
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
        m = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        v = torch.zeros_like(m)
        for name, d in st["state"].items():
            s = self.by_name.get(name)
            if s is None:
                continue
            sl = slice(s.offset, s.offset + s.numel)
            m[sl].copy_(d["exp_avg"].reshape(-1))
            v[sl].copy_(d["exp_avg_sq"].reshape(-1))
        self._scatter_full(m, self.m)
        self._scatter_full(v, self.v)

    def _state_ranges(self, everything_local: bool) -> list:
        out = []
        st = self.shard_total
        for u in [self.root] + self.ring_units:
            a = u.lo + u.per * self.rank
            b = min(a + u.per, u.hi)
            if b > a:
                for kind, buf in (("p", self.p32), ("m", self.m), ("v", self.v)):
                    out.append((kind, a, b, buf[u.soff:u.soff + (b - a)]))
        n_ep = self.ep_end - self.decay_end
        if n_ep:
            for kind, buf in (("p", self.p32), ("m", self.m), ("v", self.v)):
                out.append((kind, self.decay_end, self.ep_end, buf[st:st + n_ep]))
        if self.total > self.ep_end and (everything_local or self.rank == 0):
            for kind, buf in (("p", self.p32), ("m", self.m), ("v", self.v)):
                out.append((kind, self.ep_end, self.total, buf[st + n_ep:]))
        return out

    def export_state_ranges(self) -> list:
        return self._state_ranges(everything_local=False)

    def import_state_ranges(self) -> list:
        return self._state_ranges(everything_local=True)

    def memory_report(self) -> dict:
        """Bytes this rank holds per category (what the sharding buys is persistent state / world)."""
        return {"persistent_sharded_state": int(self.shard_total * (4 * 4 + 2)),
                "persistent_local_state": int((self.total - self.decay_end) * (4 * 3 + 2)),
                "staging_bf16": int(self.p16.numel() * 2), "staging_grad_fp32": int(self.g32.numel() * 4),
                "replicated_equivalent": int(self.total * (4 * 4 + 2))}
