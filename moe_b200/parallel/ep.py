"""Expert parallelism: experts are sharded over the ranks of one NVLink domain; tokens travel to
the rank that owns their expert and results travel back, both as peer stores issued from inside
kernels (no NCCL all-to-all, no host synchronisation).

Per MoE layer, forward:
  1. local plan by global expert id (counts, stable rank-in-expert);
  2. `ep_exchange`: counts to every peer, identical layout computation everywhere;
  3. `ep_dispatch`: rows pushed into the owners' receive buffers + flag;
  4. grouped up-projection + SwiGLU on the receive buffer: its producer warp waits for the senders'
     flags, TMA reads only local memory;
  5. grouped down-projection whose epilogue stores each result row into the token owner's return
     buffer and posts a flag when the whole grid is done;
  6. weighted combine on the token owner, after the owners' flags.
Backward runs the same route with gradients (rows scaled by the routing weight on the way out),
weight gradients stay on the expert owner.

Receive buffers are sized for `capacity_factor` x the balanced load (at most the worst case); an
owner that is sent more rows than that refuses the step through the kernel status word.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops import gemm as G

MAX_RANKS = 8
CH_COUNTS, CH_DISPATCH, CH_RETURN = 0, 1, 2


class _Symm:
    def __init__(self, shape, dtype, device, group):
        import torch.distributed._symmetric_memory as sm

        self.t = sm.empty(*shape, dtype=dtype, device=device)
        self.t.zero_()
        torch.cuda.synchronize(device)
        self.h = sm.rendezvous(self.t, group)
        self.ptrs = [int(p) for p in self.h.buffer_ptrs]


class EPContext:
    def __init__(self, num_experts: int, group=None, device=None, capacity_factor: float = 2.0):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > MAX_RANKS:
            raise ValueError("expert parallelism over peer memory supports at most 8 ranks")
        if num_experts % self.world != 0:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.E, self.El = num_experts, num_experts // self.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.capacity_factor = capacity_factor
        self.ext = _ext.load()
        self.flags = _Symm((3 * MAX_RANKS,), torch.int32, self.device, self.group)
        self.cmat = _Symm((self.world * self.E,), torch.int32, self.device, self.group)
        self.epoch_base = torch.ones(1, dtype=torch.int32, device=self.device)
        self.used = 0
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.gemm_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = G.status_word(self.device)
        self._bufs: dict = {}
        self.call_index = 0
        # call-site identity: the decoder layer sets `site` before it runs (also when a checkpointed layer is
        # recomputed), so forward and recomputation of one layer find the same buffers
        self.site: int | None = None
        # with activation checkpointing a layer's buffers are rewritten by its recomputation right before
        # its backward, so two alternating sets serve every layer
        self.share_buffers = False

    # ------------------------------------------------------------------ bookkeeping
    def begin_step(self) -> None:
        self.call_index = 0

    def next_epoch(self) -> int:
        off = self.used
        self.used += 1
        return off

    def end_step(self) -> None:
        """Advance the epoch base on the device (part of a captured graph, so replays keep counting)."""
        if self.used:
            self.epoch_base.add_(self.used)
            self.used = 0

    def capacity(self, T: int, K: int) -> int:
        worst = self.world * T * K
        cap = min(worst, int(self.capacity_factor * T * K)) + self.El * 128
        return (cap + 127) // 128 * 128

    def buffers(self, key, T: int, K: int, H: int) -> dict:
        """Symmetric buffers of one MoE call site (`key`), allocated collectively on first use."""
        k = (key, T, K, H)
        b = self._bufs.get(k)
        if b is None:
            cap = self.capacity(T, K)
            mk = lambda shape, dt: _Symm(shape, dt, self.device, self.group)
            b = {"cap": cap, "xrecv": mk((cap, H), torch.bfloat16), "meta": mk((cap,), torch.int32),
                 "yret": mk((T * K, H), torch.bfloat16)}
            self._bufs[k] = b
        return b

    def bwd_buffers(self, parity: int, T: int, K: int, H: int) -> dict:
        k = ("bwd", parity, T, K, H)
        b = self._bufs.get(k)
        if b is None:
            cap = self.capacity(T, K)
            mk = lambda shape, dt: _Symm(shape, dt, self.device, self.group)
            b = {"dyrecv": mk((cap, H), torch.bfloat16), "dxret": mk((T * K, H), torch.bfloat16)}
            self._bufs[k] = b
        return b

    def local_flags(self, chan: int) -> torch.Tensor:
        return self.flags.t[chan * MAX_RANKS:(chan + 1) * MAX_RANKS]

    def wait_kw(self, chan: int, epoch_off: int) -> dict:
        return dict(ep_wait_flags=self.local_flags(chan), ep_wait_n=self.world, ep_epoch_base=self.epoch_base,
                    ep_wait_epoch_off=epoch_off)

    def scatter_kw(self, dst_ptrs, meta: torch.Tensor, epoch_off: int) -> dict:
        return dict(ep_scatter_dst=dst_ptrs, ep_scatter_meta=meta, ep_post_flags=self.flags.ptrs,
                    ep_post_index=CH_RETURN * MAX_RANKS + self.rank, ep_post_epoch_off=epoch_off,
                    ep_world=self.world, ep_counter=self.gemm_counter, ep_epoch_base=self.epoch_base)


class EPMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, gate_up, down, ep: EPContext):
        from ..ops.functional import BF16, MoEPlan, w16

        e = ep.ext
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        T, H = x2.shape
        K = topk_idx.shape[-1]
        w1, w2 = w16(gate_up), w16(down)
        El, I2, _ = w1.shape
        I = I2 // 2
        dev = x2.device
        idx32 = topk_idx.reshape(T, K).to(torch.int32).contiguous()
        tw = topk_w.reshape(T, K).float().contiguous()
        plan = MoEPlan(idx32, ep.E)  # by global expert id: counts + stable rank inside each expert
        key = ep.site if ep.site is not None else ep.call_index
        ep.call_index += 1
        if ep.share_buffers:
            key &= 1
        b = ep.buffers(key, T, K, H)
        cap = b["cap"]
        send_base = torch.empty(ep.E, dtype=torch.int32, device=dev)
        rseg = torch.empty(El + 1, dtype=torch.int32, device=dev)
        rtile = torch.empty(cap // 128, dtype=torch.int32, device=dev)
        rnt = torch.empty(1, dtype=torch.int32, device=dev)
        # the received rows as pair tiles, for the pair-tile GEMM kernels
        rpair = torch.empty((cap // 128 + El + 1) // 2, 2, dtype=torch.int32, device=dev)
        rnp = torch.empty(1, dtype=torch.int32, device=dev)
        pair = (rpair, rnp)
        e0 = ep.next_epoch()
        e.ep_exchange(plan.counts, ep.cmat.ptrs, ep.flags.ptrs, ep.epoch_base, e0, ep.rank, ep.world, ep.E, H,
                      send_base, rseg, rtile, rnt, b["xrecv"].t, b["meta"].t, ep.status, rpair, rnp)
        e1 = ep.next_epoch()
        e.ep_dispatch(x2, None, idx32.view(-1), plan.pos, plan.seg_off, send_base, b["xrecv"].ptrs, b["meta"].ptrs,
                      ep.flags.ptrs, ep.epoch_base, e1, ep.rank, ep.world, ep.E, K, cap, ep.counter)
        act = torch.empty(cap, I, dtype=BF16, device=dev)
        gu = torch.empty(cap, I2, dtype=BF16, device=dev)
        G.grouped_up_swiglu(b["xrecv"].t, w1, rtile, rnt, act, gu, ep=ep.wait_kw(CH_DISPATCH, e1), pair=pair)
        e2 = ep.next_epoch()
        G.grouped_nt(act, w2, rtile, rnt, b["yret"].t, scatter=True, ep=ep.scatter_kw(b["yret"].ptrs, b["meta"].t, e2))
        out = torch.empty(T, H, dtype=BF16, device=dev)
        e.moe_combine(b["yret"].t, None, tw, None, out, K, ep.local_flags(CH_RETURN), ep.world, ep.epoch_base, e2,
                      ep.status)
        ctx.save_for_backward(gu, act, tw, idx32, send_base, rseg, rtile, rnt, rpair, rnp)
        ctx.plan, ctx.ep, ctx.bufs, ctx.key = plan, ep, b, key
        ctx.params, ctx.w = (gate_up, down), (w1, w2)
        ctx.in_shape = tuple(x.shape)
        return out.view(ctx.in_shape)

    @staticmethod
    def backward(ctx, dout):
        from ..ops.functional import BF16, GradSink

        gu, act, tw, idx32, send_base, rseg, rtile, rnt, rpair, rnp = ctx.saved_tensors
        ep, b, plan = ctx.ep, ctx.bufs, ctx.plan
        e = ep.ext
        w1, w2 = ctx.w
        gate_up, down = ctx.params
        T, K = idx32.shape
        H = b["xrecv"].t.shape[1]
        cap = b["cap"]
        dev = gu.device
        d2 = dout.reshape(T, H)
        d2 = (d2 if d2.dtype == BF16 else d2.to(BF16)).contiguous()
        # gradient of the routing weights: <dout[t], y[t, k]> with the unscaled expert outputs kept from forward
        dw = torch.empty(T, K, dtype=torch.float32, device=dev)
        e.moe_slot_dot(d2, b["yret"].t, K, dw)
        bb = ep.bwd_buffers(ctx.key & 1, T, K, H)
        e3 = ep.next_epoch()
        e.ep_dispatch(d2, tw.view(-1), idx32.view(-1), plan.pos, plan.seg_off, send_base, bb["dyrecv"].ptrs,
                      b["meta"].ptrs, ep.flags.ptrs, ep.epoch_base, e3, ep.rank, ep.world, ep.E, K, cap, ep.counter)
        dgu = torch.empty_like(gu)
        G.grouped_nn_swiglu_bwd(bb["dyrecv"].t, w2, rtile, rnt, gu, dgu, ep=ep.wait_kw(CH_DISPATCH, e3),
                                pair=(rpair, rnp))
        s2 = GradSink(down)
        t2, b2 = s2.target()
        G.grouped_tn(bb["dyrecv"].t, act, rseg, t2, beta=b2)
        e4 = ep.next_epoch()
        G.grouped_nn(dgu, w1, rtile, rnt, bb["dxret"].t, scatter=True,
                     ep=ep.scatter_kw(bb["dxret"].ptrs, b["meta"].t, e4))
        s1 = GradSink(gate_up)
        t1, b1 = s1.target()
        G.grouped_tn(dgu, b["xrecv"].t, rseg, t1, beta=b1)
        dx = torch.empty(T, H, dtype=BF16, device=dev)
        e.moe_combine(bb["dxret"].t, None, None, None, dx, K, ep.local_flags(CH_RETURN), ep.world, ep.epoch_base, e4,
                      ep.status)
        return dx.view(ctx.in_shape), dw, None, s1.done(t1), s2.done(t2), None


def moe_experts_ep(x, topk_idx, topk_w, gate_up, down, ep: EPContext):
    return EPMoEFn.apply(x, topk_w, topk_idx, gate_up, down, ep)
