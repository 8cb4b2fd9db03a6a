"""Symmetric (peer-mapped) buffers for the NVLink kernels, and the fused gradient all-reduce.

Each rank allocates the same buffers through `torch.distributed._symmetric_memory`; after the
rendezvous every rank holds device pointers to every peer's copy (and, on NVSwitch systems, one
multicast address that fans a store out to all ranks and reduces a load across them).  The kernels
in `csrc/comm` use those pointers with ordinary peer loads / stores or `multimem` instructions;
nothing here goes through TMA.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

MAX_RANKS = 8
CANARY = 1.2345678e30  # guard-word value of the debug mode


class PeerBuffers:
    """Three symmetric allocations: the flat fp32 gradient buffer, flag words, squared-norm slots."""

    def __init__(self, numel: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as sm

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"the peer-memory kernels support at most {MAX_RANKS} ranks (one NVLink domain)")
        # Debug aid (MOE_B200_DEBUG_CANARY=1): guard words on both sides of the gradient buffer, which peers write
        # into; `check_canaries()` (called by the engine after every step in that mode) reports an overrun.
        self._guard = 64 if os.environ.get("MOE_B200_DEBUG_CANARY", "0") == "1" else 0
        self._grad_full = sm.empty(numel + 2 * self._guard, dtype=torch.float32, device=device)
        self.grad = self._grad_full[self._guard:self._guard + numel]
        self.flags = sm.empty(4 * MAX_RANKS, dtype=torch.int32, device=device)
        self.norm = sm.empty(MAX_RANKS, dtype=torch.float32, device=device)
        for t in (self._grad_full, self.flags, self.norm):
            t.zero_()
        if self._guard:
            self._grad_full[:self._guard] = CANARY
            self._grad_full[-self._guard:] = CANARY
        torch.cuda.synchronize(device)
        hg = sm.rendezvous(self._grad_full, group)
        hf = sm.rendezvous(self.flags, group)
        hn = sm.rendezvous(self.norm, group)
        self._handles = (hg, hf, hn)
        self.grad_ptrs = [int(p) + 4 * self._guard for p in hg.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in hf.buffer_ptrs]
        self.norm_ptrs = [int(p) for p in hn.buffer_ptrs]
        mc = 0
        try:
            if hg.has_multicast_support(device.type, device.index if device.index is not None else 0):
                mc = int(hg.multicast_ptr)
        except Exception:
            mc = int(getattr(hg, "multicast_ptr", 0) or 0)
        if mc:
            mc += 4 * self._guard
        # NVLS only on request to opt out: MOE_B200_MULTIMEM=0 forces plain peer loads / stores
        self.multicast_ptr = mc if os.environ.get("MOE_B200_MULTIMEM", "1") != "0" else 0
        self.group = group
        self.p16 = None
        self.p16_ptrs: list[int] = []
        self.p16_mc = 0  # multicast address of the bf16 parameter copy (0: peer stores)
        dist.barrier(group)
        # Measurement aid: MOE_B200_COMM_STUB=1 points every "peer" at this rank's own buffers and pre-sets the
        # flag words, so the same kernels run with the same local work but nothing crosses NVLink and nobody
        # waits for anybody.  Step time minus the stubbed step time is the exposed communication.  Results of a
        # stubbed run are not a data-parallel average and must not be trained on.
        self.stubbed = os.environ.get("MOE_B200_COMM_STUB", "0") == "1"
        if self.stubbed:
            self.grad_ptrs = [self.grad_ptrs[self.rank]] * self.world
            self.flag_ptrs = [self.flag_ptrs[self.rank]] * self.world
            self.norm_ptrs = [self.norm_ptrs[self.rank]] * self.world
            self.multicast_ptr = 0
            self.flags.fill_(1 << 30)
            torch.cuda.synchronize(device)

    def check_canaries(self) -> None:
        """Raises if anything wrote outside the gradient buffer (debug mode only; synchronises)."""
        if not self._guard:
            return
        g = self._guard
        lo, hi = self._grad_full[:g], self._grad_full[-g:]
        if not (bool((lo == CANARY).all()) and bool((hi == CANARY).all())):
            raise RuntimeError("guard words around the symmetric gradient buffer were overwritten "
                               f"(rank {self.rank}: below {int((lo != CANARY).sum())}, above {int((hi != CANARY).sum())})")

    def add_param_copy(self, numel: int) -> None:
        """A symmetric bf16 parameter copy: with a sharded optimizer the owner of a slice stores the updated
        weights into every rank's copy."""
        import torch.distributed._symmetric_memory as sm

        self.p16 = sm.empty(numel, dtype=torch.bfloat16, device=self.grad.device)
        self.p16.zero_()
        torch.cuda.synchronize(self.grad.device)
        h = sm.rendezvous(self.p16, self.group)
        self._handles = self._handles + (h,)
        self.p16_ptrs = [int(p) for p in h.buffer_ptrs]
        if self.multicast_ptr:  # NVLS in use for the gradients: publish the weights through the switch as well
            try:
                self.p16_mc = int(getattr(h, "multicast_ptr", 0) or 0)
            except Exception:
                self.p16_mc = 0
        if getattr(self, "stubbed", False):
            self.p16_ptrs = [self.p16_ptrs[self.rank]] * self.world
            self.p16_mc = 0
        dist.barrier(self.group)


class FusedAllReduce:
    """Launches `csrc/comm/allreduce.cu` on slices of a flat gradient buffer (see that file)."""

    def __init__(self, ext, grad_ptrs, flag_ptrs, norm_ptrs, multicast_ptr, rank, world, device, status,
                 blocks: int = 128, limit_ns: int = 0):
        self.ext, self.rank, self.world = ext, rank, world
        self.grad_ptrs, self.flag_ptrs, self.norm_ptrs, self.mc = grad_ptrs, flag_ptrs, norm_ptrs, multicast_ptr
        self.state_i = torch.zeros(2, dtype=torch.int32, device=device)
        self.state_f = torch.zeros(2 + 148, dtype=torch.float32, device=device)  # running sum + per-block partials
        self.epoch_base = torch.ones(1, dtype=torch.int32, device=device)
        self.status = status
        # CTAs of the reduce kernel: enough loads in flight for NVLink, few enough to leave the SMs to backward
        self.blocks, self.limit_ns = int(os.environ.get("MOE_B200_AR_BLOCKS", blocks)), limit_ns
        self.launched = 0  # buckets since the last `end_step`
        self._scratch_f = None

    def reduce(self, off: int, n: int, final_bucket: bool, publish: bool = True, count_norm: bool = True) -> None:
        """`count_norm=False`: the bucket's squared norm goes to a scratch accumulator (the caller accounts for
        these gradients itself, e.g. after adding several micro-batches' reduced slices)."""
        if not count_norm and final_bucket:
            raise ValueError("the final bucket publishes the norm and must count")
        if not count_norm and self._scratch_f is None:
            self._scratch_f = torch.zeros_like(self.state_f)
        self.ext.allreduce(self.grad_ptrs, self.flag_ptrs, self.norm_ptrs, self.mc, self.rank, self.world, off, n,
                           1.0 / self.world, self.epoch_base, self.launched, final_bucket, publish, self.mc != 0,
                           self.blocks, self.state_i, self.state_f if count_norm else self._scratch_f, self.status,
                           self.limit_ns)
        self.launched += 1

    def param_barrier(self) -> None:
        """All ranks' parameter stores into this rank's memory are complete once this kernel has run."""
        self.ext.peer_barrier(self.flag_ptrs, self.rank, self.world, 2, self.epoch_base, self.launched, self.status)
        self.launched += 1

    def end_step(self) -> None:
        """Advance the epoch base on the device (captured by a CUDA graph, so replays keep counting)."""
        if self.launched:
            self.epoch_base.add_(self.launched)
            self.launched = 0
