"""Autograd wrappers around the sm_100a kernels (the CUDA execution path).

Weights are `torch.nn.Parameter`s holding the fp32 master values.  When the
training engine has attached a bf16 compute copy (`p._bf16`) and an fp32
gradient accumulator (`p.main_grad`), forward reads the copy and backward lets
the weight-gradient GEMM epilogue write or accumulate straight into
`main_grad` (first write of a step overwrites, later ones accumulate,
tracked by `p._grad_live`) and returns no gradient tensor.  Without an
engine the same functions cast on the fly and return ordinary gradients.
"""
from __future__ import annotations

import math
import os

import torch

from . import _ext
from . import gemm as G

BF16 = torch.bfloat16


def ext():
    return _ext.load()


# ------------------------------------------------------------ parameter access
def w16(p: torch.Tensor) -> torch.Tensor:
    c = getattr(p, "_bf16", None)
    return c if c is not None else p.detach().to(BF16)


def w32(p: torch.Tensor) -> torch.Tensor:
    return p.detach() if p.dtype == torch.float32 else p.detach().float()


class GradSink:
    """Where a weight gradient goes: the engine's fp32 accumulator, or a fresh tensor."""

    def __init__(self, p: torch.Tensor):
        self.p = p
        self.main = getattr(p, "main_grad", None)

    def target(self) -> tuple[torch.Tensor, int]:
        """Returns (fp32 tensor to write, beta)."""
        if self.main is not None:
            beta = 1 if getattr(self.p, "_grad_live", False) else 0
            return self.main, beta
        return torch.empty(self.p.shape, dtype=torch.float32, device=self.p.device), 0

    def done(self, t: torch.Tensor):
        """Value to return from autograd.backward for this parameter."""
        if self.main is not None:
            self.p._grad_live = True
            return None
        return t.to(self.p.dtype)


def _scratch(name: str, numel: int, dtype, device) -> torch.Tensor:
    key = (name, dtype, device)
    t = _SCRATCH.get(key)
    if t is None or t.numel() < numel:
        t = torch.empty(max(numel, 1), dtype=dtype, device=device)
        _SCRATCH[key] = t
    return t


_SCRATCH: dict = {}


# ------------------------------------------------------------------- embedding
class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        table = w16(weight)
        flat = ids.reshape(-1).contiguous()
        out = torch.empty(flat.numel(), table.shape[1], dtype=BF16, device=table.device)
        e = ext()
        e.embed_fwd(flat, table, out)
        ctx.sorted = None
        n = flat.numel()
        if ctx.needs_input_grad[1] and n <= e.embed_sort_capacity():
            # the backward pass needs the (id, position) keys sorted; the ids are known now, so the one-block
            # sort runs on a side stream under the forward pass instead of in the tail of backward
            dev = flat.device
            main, side = torch.cuda.current_stream(dev), _side_stream(dev)
            keys = torch.empty(n, dtype=torch.int64, device=dev)
            ready = torch.cuda.Event()
            ready.record(main)
            done = torch.cuda.Event()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                e.embed_sort(flat, table.shape[0], keys)
                done.record(side)
            ctx.sorted = (keys, done)  # kept alive until backward has waited for `done` on the main stream
        ctx.save_for_backward(flat)
        ctx.weight = weight
        ctx.shape = tuple(ids.shape)
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        e = ext()
        sink = GradSink(ctx.weight)
        tgt, beta = sink.target()
        if beta == 0:
            tgt.zero_()
        n = flat.numel()
        # deterministic: (id, position) keys are sorted and each id's rows are added in position order
        if ctx.sorted is not None:
            keys, done = ctx.sorted
            torch.cuda.current_stream(flat.device).wait_event(done)
            presorted = True
        elif n <= e.embed_sort_capacity():
            keys = _scratch("embed_keys", n, torch.int64, flat.device)
            presorted = False
        else:  # beyond the single-block sort: library radix sort of the same keys
            V = tgt.shape[0]
            big = torch.iinfo(torch.int64).max
            k = torch.where((flat >= 0) & (flat < V), (flat << 32) | torch.arange(n, device=flat.device),
                            torch.full_like(flat, big))
            keys = torch.sort(k).values  # invalid ids last ...
            keys = torch.where(keys == big, torch.full_like(keys, -1), keys).contiguous()  # ... as all-ones keys
            presorted = True
        e.embed_bwd(flat, dout.reshape(n, -1).contiguous(), tgt, keys, presorted, True)
        return None, sink.done(tgt)


# --------------------------------------------------------------------- rmsnorm
class RMSNormFn(torch.autograd.Function):
    """y = rmsnorm(x [+ res]); returns (h, y) where h = x + res is the new residual stream."""

    @staticmethod
    def forward(ctx, x, res, weight, eps):
        x = x.contiguous()
        H = x.shape[-1]
        T = x.numel() // H
        w = w32(weight)
        y = torch.empty_like(x)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        if res is not None:
            h = torch.empty_like(x)
            ext().rmsnorm_fwd(x, res.contiguous(), w, h, y, rstd, eps)
        else:
            h = x
            ext().rmsnorm_fwd(x, None, w, None, y, rstd, eps)
        ctx.save_for_backward(h, rstd)
        ctx.weight = weight
        ctx.has_res = res is not None
        return h, y

    @staticmethod
    def backward(ctx, dh, dy):
        h, rstd = ctx.saved_tensors
        H = h.shape[-1]
        T = h.numel() // H
        e = ext()
        sink = GradSink(ctx.weight)
        tgt, beta = sink.target()
        part = _scratch("rms_dw", e.rmsnorm_bwd_blocks(T) * H, torch.float32, h.device)
        dx = torch.empty_like(h)
        dres = dh.contiguous() if dh is not None else None
        e.rmsnorm_bwd(dy.contiguous(), h, rstd, w32(ctx.weight), dres, dx, part, tgt.view(-1), bool(beta))
        return dx, (dx if ctx.has_res else None), sink.done(tgt), None


def rmsnorm(x, weight, eps):
    _, y = RMSNormFn.apply(x, None, weight, eps)
    return y


def add_rmsnorm(x, res, weight, eps):
    """(x + res, rmsnorm(x + res)) in one pass."""
    return RMSNormFn.apply(x, res, weight, eps)


# ---------------------------------------------------------------------- linear
class LinearFn(torch.autograd.Function):
    """y = x @ W^T with W given as one or several row-adjacent parameters (e.g. q, k, v projections)."""

    @staticmethod
    def forward(ctx, x, fused, rope, *weights):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if x2.dtype != BF16:
            x2 = x2.to(BF16)
        x2 = x2.contiguous()
        if fused is not None:
            wmat = fused[0]
        elif len(weights) == 1:
            wmat = w16(weights[0])
        else:
            wmat = torch.cat([w16(w) for w in weights], dim=0)
        if rope is not None and rope.usable(x2.shape[0], wmat.shape[0], K):
            # QKV projection: the per-head RMSNorm + RoPE of q and k runs in the GEMM's epilogue; the raw projection
            # (this function's output, what the norm's backward needs) is written beside the rotated one
            cs = rope_table(rope.S, rope.hd, rope.theta, x2.device)
            y, rope.rot, rope.rstd = G.gemm_nt_qkrope(x2, wmat, cs, w32(rope.q_w), w32(rope.k_w), rope.S, rope.nh,
                                                      rope.nkv, rope.eps)
            rope.cs = cs
        else:
            y = G.gemm_nt(x2, wmat)
        ctx.save_for_backward(x2)
        ctx.wmat = wmat
        ctx.fused = fused
        ctx.weights = weights
        ctx.in_shape = tuple(x.shape)
        return y.view(*x.shape[:-1], wmat.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        wmat = ctx.wmat
        N, K = wmat.shape
        dy2 = dy.reshape(-1, N)
        if dy2.dtype != BF16:
            dy2 = dy2.to(BF16)
        dy2 = dy2.contiguous()
        dx = G.gemm_nn(dy2, wmat).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        weights = ctx.weights
        if ctx.fused is not None:
            grad_view = ctx.fused[1]
            beta = 1 if all(getattr(w, "_grad_live", False) for w in weights) else 0
            if beta == 0 and any(getattr(w, "_grad_live", False) for w in weights):
                raise RuntimeError("fused weight group has inconsistent gradient state")
            G.gemm_tn(dy2, x2, grad_view, beta=beta)
            for w in weights:
                w._grad_live = True
            return (dx, None, None) + (None,) * len(weights)
        if len(weights) == 1:
            sink = GradSink(weights[0])
            tgt, beta = sink.target()
            G.gemm_tn(dy2, x2, tgt, beta=beta)
            return dx, None, None, sink.done(tgt)
        full = torch.empty(N, K, dtype=torch.float32, device=dy2.device)
        G.gemm_tn(dy2, x2, full)
        outs, r = [], 0
        for w in weights:
            n = w.shape[0]
            piece = full[r:r + n]
            r += n
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                if getattr(w, "_grad_live", False):
                    mg.add_(piece)
                else:
                    mg.copy_(piece)
                w._grad_live = True
                outs.append(None)
            else:
                outs.append(piece.to(w.dtype))
        return (dx, None, None, *outs)


def linear(x, *weights, fused=None):
    return LinearFn.apply(x, fused, None, *weights)


class RopeSpec:
    """What the QKV projection needs to apply QK-norm + RoPE in its epilogue, and where it leaves the results."""

    def __init__(self, q_w, k_w, B, S, nh, nkv, hd, theta, eps):
        self.q_w, self.k_w = q_w, k_w
        self.B, self.S, self.nh, self.nkv, self.hd, self.theta, self.eps = B, S, nh, nkv, hd, theta, eps
        self.rot = self.rstd = self.cs = None

    def usable(self, M: int, N: int, K: int) -> bool:
        return (M == self.B * self.S and N == (self.nh + 2 * self.nkv) * self.hd
                and G.qkv_rope_supported(M, N, K, self.hd))


def qkv_proj_norm_rope(x, wq, wk, wv, fused, q_norm_w, k_norm_w, B, S, nh, nkv, hd, theta, eps):
    """(q, k, v) `[B,S,h,hd]` from the hidden states: fused QKV projection, per-head RMSNorm of q and k, RoPE.
    Where the pair-tile GEMM applies (head_dim 128) norm and rotation run in the projection's epilogue and q, k, v
    are slices of one `[B*S, (nh + 2 nkv) * hd]` buffer; otherwise a separate kernel follows the GEMM."""
    spec = RopeSpec(q_norm_w, k_norm_w, B, S, nh, nkv, hd, theta, eps)
    qkv = LinearFn.apply(x, fused, spec, wq, wk, wv)
    return QKNormRopeFn.apply(qkv, q_norm_w, k_norm_w, B, S, nh, nkv, hd, theta, eps, spec if spec.rot is not None else None)


# ------------------------------------------------------------ dense SwiGLU MLP
class SwiGLUMLPFn(torch.autograd.Function):
    """`down(silu(gate(x)) * up(x))`: the gate|up projection is one GEMM whose epilogue applies SwiGLU, the
    input-gradient GEMM of the down projection applies its derivative (same epilogues as the expert path)."""

    @staticmethod
    def forward(ctx, x, gate_w, up_w, down_w, fused):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if x2.dtype != BF16:
            x2 = x2.to(BF16)
        x2 = x2.contiguous()
        T = x2.shape[0]
        wgu = fused[0] if fused is not None else torch.cat([w16(gate_w), w16(up_w)], dim=0)
        wd = w16(down_w)
        I = wgu.shape[0] // 2
        act = torch.empty(T, I, dtype=BF16, device=x2.device)
        gu = torch.empty(T, 2 * I, dtype=BF16, device=x2.device)
        G.dense_up_swiglu(x2, wgu, act, gu)
        y = G.gemm_nt(act, wd)
        ctx.save_for_backward(x2, gu, act)
        ctx.w = (wgu, wd)
        ctx.params = (gate_w, up_w, down_w)
        ctx.fused = fused
        ctx.in_shape = tuple(x.shape)
        return y.view(*x.shape[:-1], wd.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, gu, act = ctx.saved_tensors
        wgu, wd = ctx.w
        gate_w, up_w, down_w = ctx.params
        T, H = x2.shape
        dy2 = dy.reshape(T, -1)
        if dy2.dtype != BF16:
            dy2 = dy2.to(BF16)
        dy2 = dy2.contiguous()
        dgu = torch.empty_like(gu)
        G.dense_swiglu_bwd(dy2, wd, gu, dgu)
        sd = GradSink(down_w)
        td, bd = sd.target()
        G.gemm_tn(dy2, act, td, beta=bd)
        dx = G.gemm_nn(dgu, wgu).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        I = wgu.shape[0] // 2
        if ctx.fused is not None:
            live = [getattr(w, "_grad_live", False) for w in (gate_w, up_w)]
            if live[0] != live[1]:
                raise RuntimeError("fused gate/up weights have inconsistent gradient state")
            G.gemm_tn(dgu, x2, ctx.fused[1], beta=1 if live[0] else 0)
            gate_w._grad_live = up_w._grad_live = True
            return dx, None, None, sd.done(td), None
        full = torch.empty(2 * I, H, dtype=torch.float32, device=x2.device)
        G.gemm_tn(dgu, x2, full)
        outs = []
        for w, piece in ((gate_w, full[:I]), (up_w, full[I:])):
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                mg.add_(piece) if getattr(w, "_grad_live", False) else mg.copy_(piece)
                w._grad_live = True
                outs.append(None)
            else:
                outs.append(piece.to(w.dtype))
        return dx, outs[0], outs[1], sd.done(td), None


def swiglu_mlp(x, gate_w, up_w, down_w, fused_gate_up=None):
    return SwiGLUMLPFn.apply(x, gate_w, up_w, down_w, fused_gate_up)


# ------------------------------------------------------------ qk-norm + rope
_ROPE_TABLES: dict = {}


def rope_table(S: int, hd: int, theta: float, device) -> torch.Tensor:
    """Interleaved (cos, sin) table `[S, hd/2, 2]` in fp32."""
    key = (S, hd, float(theta), device)
    t = _ROPE_TABLES.get(key)
    if t is None:
        inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32, device=device) / hd))
        fr = torch.outer(torch.arange(S, dtype=torch.float32, device=device), inv)
        t = torch.stack([fr.cos(), fr.sin()], dim=-1).contiguous()
        _ROPE_TABLES[key] = t
    return t


class QKNormRopeFn(torch.autograd.Function):
    """Fused QKV projection output -> (q, k, v) in `[B, S, heads, hd]`, with per-head RMSNorm and RoPE on q, k."""

    @staticmethod
    def forward(ctx, qkv, q_w, k_w, B, S, nh, nkv, hd, theta, eps, pre=None):
        qkv2 = qkv.reshape(B * S, (nh + 2 * nkv) * hd).contiguous()
        T = B * S
        dev = qkv2.device
        if pre is not None:  # already computed by the projection's epilogue (`RopeSpec`): hand out the slices
            cs, rstd = pre.cs, pre.rstd.view(-1)
            q, k, v = pre.rot.view(B, S, nh + 2 * nkv, hd).split([nh, nkv, nkv], dim=2)
        else:
            cs = rope_table(S, hd, theta, dev)
            q = torch.empty(B, S, nh, hd, dtype=BF16, device=dev)
            k = torch.empty(B, S, nkv, hd, dtype=BF16, device=dev)
            v = torch.empty(B, S, nkv, hd, dtype=BF16, device=dev)
            rstd = torch.empty(T * (nh + nkv), dtype=torch.float32, device=dev)
            ext().qknorm_rope_fwd(qkv2, w32(q_w), w32(k_w), cs, q, k, v, rstd, S, nh, nkv, hd, eps)
        ctx.save_for_backward(qkv2, rstd, cs)
        ctx.q_w, ctx.k_w = q_w, k_w
        ctx.dims = (B, S, nh, nkv, hd)
        ctx.qkv_shape = tuple(qkv.shape)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv2, rstd, cs = ctx.saved_tensors
        B, S, nh, nkv, hd = ctx.dims
        T = B * S
        e = ext()
        dev = qkv2.device
        if dq is None:
            dq = torch.zeros(B, S, nh, hd, dtype=BF16, device=dev)
        if dk is None:
            dk = torch.zeros(B, S, nkv, hd, dtype=BF16, device=dev)
        if dv is None:
            dv = torch.zeros(B, S, nkv, hd, dtype=BF16, device=dev)
        sq, sk = GradSink(ctx.q_w), GradSink(ctx.k_w)
        tq, bq = sq.target()
        tk, bk = sk.target()
        if bq != bk:  # keep one accumulate flag for the fused kernel
            (tq if bq == 0 else tk).zero_()
            bq = bk = 1
        part = _scratch("qk_dw", e.qknorm_rope_blocks(T) * 2 * hd, torch.float32, dev)
        dqkv = torch.empty_like(qkv2)
        e.qknorm_rope_bwd(dq.contiguous(), dk.contiguous(), dv.contiguous(), qkv2, rstd, w32(ctx.q_w), w32(ctx.k_w), cs,
                          dqkv, part, tq, tk, bool(bq), S, nh, nkv, hd)
        return dqkv.view(ctx.qkv_shape), sq.done(tq), sk.done(tk), None, None, None, None, None, None, None, None


def qk_norm_rope(qkv, q_w, k_w, B, S, nh, nkv, hd, theta, eps):
    return QKNormRopeFn.apply(qkv, q_w, k_w, B, S, nh, nkv, hd, theta, eps, None)


# ------------------------------------------------------------------- attention
def _sdpa(q, k, v):
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True)
    return o.transpose(1, 2).contiguous()


def flash_supported(q, k) -> bool:
    """Shapes the tcgen05 kernels cover: head_dim 128 or 64, length a multiple of 128, an even number of
    query heads per key/value head (a CTA works on two query heads that share their key/value tiles)."""
    B, S, nh, hd = q.shape
    nkv = k.shape[2]
    return (q.is_cuda and q.dtype == BF16 and hd in (128, 64) and S % 128 == 0 and nh % nkv == 0
            and (nh // nkv) % 2 == 0)


_ATTN_STATE = {"library_backward_ok": None, "dummy": {}}


def _rows4(t: torch.Tensor) -> torch.Tensor:
    """`[B,S,h,hd]` as the attention kernels take it: heads contiguous per token, tokens evenly spaced (a slice of
    the fused QKV activation qualifies as it is); anything else is made contiguous."""
    B, S, h, hd = t.shape
    ok = (t.stride(3) == 1 and t.stride(2) == hd and t.stride(1) % 8 == 0 and t.stride(1) >= h * hd
          and (B == 1 or t.stride(0) == S * t.stride(1)) and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


class FlashAttnFn(torch.autograd.Function):
    """Causal GQA attention.  Forward: `csrc/attn/flash_fwd.cu` (returns the base-2 log-sum-exp per row).
    Backward: `csrc/attn/flash_bwd.cu` (delta, dQ and dK/dV kernels).  MOE_B200_ATTN_BWD=library switches
    the backward to the cuDNN flash-attention kernel, which takes the forward's output and natural-log
    log-sum-exp as inputs (about 1.4x faster than the own kernels at B=8, S=2048, 16/8 heads); if that
    entry point is not usable in the running torch build, the gradients then come from differentiating a
    recomputed library forward."""

    @staticmethod
    def forward(ctx, q, k, v):
        B, S, nh, hd = q.shape
        q, k, v = _rows4(q), _rows4(k), _rows4(v)
        o = torch.empty(B, S, nh, hd, dtype=q.dtype, device=q.device)
        lse2 = torch.empty(B, nh, S, dtype=torch.float32, device=q.device)
        scale = 1.0 / math.sqrt(hd)
        ext().flash_fwd(q, k, v, o, lse2, scale, G.status_word(q.device))
        ctx.save_for_backward(q, k, v, o, lse2)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse2 = ctx.saved_tensors
        B, S, nh, hd = q.shape
        do = do.contiguous()
        if os.environ.get("MOE_B200_ATTN_BWD", "own") != "library":
            dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in (q, k, v))
            delta = torch.empty_like(lse2)
            ext().flash_bwd(q, k, v, o, do, lse2, delta, dq, dk, dv, ctx.scale, G.status_word(q.device))
            return dq, dk, dv
        st = _ATTN_STATE
        if st["library_backward_ok"] is not False:
            try:
                key = q.device
                if key not in st["dummy"]:
                    st["dummy"][key] = torch.zeros((), dtype=torch.int64, device=q.device)
                z = st["dummy"][key]
                lse = (lse2 * math.log(2.0)).unsqueeze(-1)
                g = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
                    do.transpose(1, 2), q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), o.transpose(1, 2),
                    lse, z, z, None, None, None, S, S, 0.0, True, scale=ctx.scale)
                st["library_backward_ok"] = True
                return g[0].transpose(1, 2), g[1].transpose(1, 2), g[2].transpose(1, 2)
            except (RuntimeError, TypeError, AttributeError) as ex:
                if st["library_backward_ok"]:
                    raise
                import warnings

                warnings.warn(f"cuDNN attention backward entry point unavailable ({ex}); recomputing through SDPA")
                st["library_backward_ok"] = False
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
            return torch.autograd.grad(_sdpa(qq, kk, vv), (qq, kk, vv), do)


def attention(q, k, v):
    """Causal GQA attention, `[B,S,h,hd]` layout.  Own forward kernel where it applies (see
    `flash_supported`), the library's scaled-dot-product attention otherwise or when
    MOE_B200_ATTN=sdpa."""
    if flash_supported(q, k) and os.environ.get("MOE_B200_ATTN", "own") != "sdpa":
        return FlashAttnFn.apply(q, k, v)
    return _sdpa(q, k, v)


# ---------------------------------------------------------------------- router
class RouterSite:
    """Where one router leaves its per-forward statistics: views into the model's stacked buffers.

    Filled by the router kernels (`csrc/moe/router.cu`): per-sequence expert counts of the actual selection
    and of the unbiased top-k, per-sequence column sums of the scores (raw and row-normalised), per-token
    score sums and top-k margins.  The balance losses are computed from these, and their gradient reaches
    the scores through `grad` (set by `AuxLossFn.backward`, read by `RouterFn.backward`), so no `[T, E]`
    gradient tensor and no one-hot tensor is ever built."""

    def __init__(self, cnt_sel, cnt_unb, psum, pn, rsum, margin, S):
        self.cnt_sel, self.cnt_unb, self.psum, self.pn = cnt_sel, cnt_unb, psum, pn
        self.rsum, self.margin, self.S = rsum, margin, S
        self.grad = None  # (g [E], d_aux [2], seq_on, seq_scale)


class RouterFn(torch.autograd.Function):
    """Router GEMM (fp32 logits) + scoring / top-k kernel.  Returns (scores fp32, weights fp32, idx int32)."""

    @staticmethod
    def forward(ctx, x, weight, bias, K, mode, norm, scale, num_groups, group_topk, site, tokens_acc, collect):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        wmat = w16(weight)
        E = wmat.shape[0]
        T = x2.shape[0]
        logits = G.gemm_nt(x2, wmat, out_dtype=torch.float32)
        scores = torch.empty(T, E, dtype=torch.float32, device=x2.device)
        tw = torch.empty(T, K, dtype=torch.float32, device=x2.device)
        ti = torch.empty(T, K, dtype=torch.int32, device=x2.device)
        b = bias.detach().float().contiguous() if bias is not None else None
        e = ext()
        if site is not None and collect:
            bt = e.router_tokens_per_block(E)
            if site.S % bt == 0:  # a block never straddles two sequences: per-block partial sums, reduced below
                nblk = T // bt
                part = _scratch("router_part", nblk * 2 * E, torch.float32, x2.device)
                e.router_fwd(logits, b, scores, tw, ti, K, mode, bool(norm), float(scale), int(num_groups or 0),
                             int(group_topk or 0), site.cnt_sel, site.cnt_unb, tokens_acc, site.rsum, site.margin,
                             part, site.S)
                e.router_part_reduce(part, site.S // bt, site.psum, site.pn)
            else:
                e.router_fwd(logits, b, scores, tw, ti, K, mode, bool(norm), float(scale), int(num_groups or 0),
                             int(group_topk or 0), site.cnt_sel, site.cnt_unb, tokens_acc, site.rsum, site.margin,
                             None, site.S)
                e.router_colsum(scores, site.rsum, site.S, site.psum, site.pn)
        else:
            e.router_fwd(logits, b, scores, tw, ti, K, mode, bool(norm), float(scale), int(num_groups or 0),
                         int(group_topk or 0))
        ctx.save_for_backward(x2, scores, ti)
        ctx.weight = weight
        ctx.wmat = wmat
        ctx.cfg = (K, mode, bool(norm), float(scale))
        ctx.in_shape = tuple(x.shape)
        ctx.site = site
        ctx.mark_non_differentiable(ti)
        return scores, tw, ti

    @staticmethod
    def backward(ctx, dscores, dtw, _):
        x2, scores, ti = ctx.saved_tensors
        K, mode, norm, scale = ctx.cfg
        T, E = scores.shape
        if dtw is None:
            dtw = torch.zeros(T, K, dtype=torch.float32, device=x2.device)
        dlogits = torch.empty(T, E, dtype=BF16, device=x2.device)
        ds = dscores.contiguous().float() if dscores is not None else None
        kw = {}
        site = ctx.site
        if site is not None and site.grad is not None:
            g, d_aux, seq_on, seq_scale = site.grad
            kw = dict(aux_g=g, d_aux=d_aux)
            if seq_on:
                kw.update(seq_cnt=site.cnt_sel, rsum=site.rsum, seq_scale=seq_scale, S=site.S)
        ext().router_bwd(ds, dtw.contiguous().float(), scores, ti, dlogits, K, mode, norm, scale, **kw)
        dx = G.gemm_nn(dlogits, ctx.wmat).view(ctx.in_shape)
        sink = GradSink(ctx.weight)
        tgt, beta = sink.target()
        G.gemm_tn(dlogits, x2, tgt, beta=beta)
        return (dx, sink.done(tgt)) + (None,) * 10


def router(x, weight, bias, K, mode, norm, scale, num_groups, group_topk, site=None, tokens_acc=None, collect=True):
    return RouterFn.apply(x, weight, bias, K, mode, norm, 1.0 if scale is None else scale, num_groups, group_topk,
                          site, tokens_acc, collect)


class MoeStatsHolder:
    """Stacked statistics buffers of all routers of a model for one forward pass (`[L, B, E]`)."""

    def __init__(self, L, B, S, E, K, device, separate_unb: bool):
        self.L, self.B, self.S, self.E, self.K = L, B, S, E, K
        self.cnt = torch.zeros(2 if separate_unb else 1, L, B, E, dtype=torch.int32, device=device)
        self.cnt_sel = self.cnt[0]
        self.cnt_unb = self.cnt[1] if separate_unb else self.cnt[0]
        self.psum = torch.zeros(L, B, E, dtype=torch.float32, device=device)
        self.pn = torch.zeros(L, B, E, dtype=torch.float32, device=device)
        self.rsum = torch.zeros(L, B * S, dtype=torch.float32, device=device)
        self.margin = torch.zeros(L, B * S, dtype=torch.float32, device=device)
        self.g = torch.zeros(E, dtype=torch.float32, device=device)
        self.out = torch.zeros(2, dtype=torch.float32, device=device)
        self.sites = [RouterSite(self.cnt_sel[l], self.cnt_unb[l], self.psum[l], self.pn[l], self.rsum[l],
                                 self.margin[l], S) for l in range(L)]

    def begin(self) -> None:
        self.cnt.zero_()
        for s in self.sites:
            s.grad = None

    def expert_counts(self) -> torch.Tensor:
        """`[L, E]` token counts by the unbiased top-k (what the routing report and the Switch loss use)."""
        return self.cnt_unb.sum(dim=1).float()


class AuxLossFn(torch.autograd.Function):
    """Switch and sequence-level balance losses from the router kernels' statistics.  Returns
    (aux, seq_aux); the gradient w.r.t. the scores is handed to the routers' backward kernels through
    their `RouterSite` (this node itself returns no tensor gradient)."""

    @staticmethod
    def forward(ctx, holder, seq_on, *scores):
        h = holder
        ext().moe_aux(h.cnt_unb, h.cnt_sel if seq_on else None, h.psum, h.pn if seq_on else None, h.K, h.S, h.g,
                      h.out)
        ctx.holder, ctx.seq_on, ctx.n = h, bool(seq_on), len(scores)
        aux, seq = h.out.unbind(0)
        return aux.clone(), seq.clone()

    @staticmethod
    def backward(ctx, d_aux, d_seq):
        h = ctx.holder
        z = torch.zeros((), dtype=torch.float32, device=h.g.device)
        pair = torch.stack([d_aux.float() if d_aux is not None else z, d_seq.float() if d_seq is not None else z])
        seq_scale = h.E / (h.K * h.S) / (h.L * h.B * h.S)
        for s in h.sites:
            s.grad = (h.g, pair, ctx.seq_on, seq_scale)
        return (None, None) + (None,) * ctx.n


def moe_aux_losses(holder, scores, seq_on: bool):
    return AuxLossFn.apply(holder, seq_on, *scores)


# --------------------------------------------------------------------- experts
def moe_capacity(T: int, K: int, E: int) -> int:
    """Rows of the expert-sorted layout in the worst case (every expert segment padded to 128)."""
    return (T * K + E * 127 + 127) // 128 * 128


class MoEPlan:
    """Device-side dispatch plan: no host synchronisation, sizes are worst-case."""

    def __init__(self, idx32: torch.Tensor, E: int):
        e = ext()
        dev = idx32.device
        T, K = idx32.shape
        self.T, self.K, self.E = T, K, E
        self.cap = moe_capacity(T, K, E)
        n = T * K
        self.counts = torch.empty(E, dtype=torch.int32, device=dev)
        self.seg_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
        self.tile_expert = torch.empty(self.cap // 128, dtype=torch.int32, device=dev)
        self.num_m_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        self.pos = torch.empty(n, dtype=torch.int32, device=dev)
        self.row_slot = torch.empty(self.cap, dtype=torch.int32, device=dev)
        # the same rows as pair tiles (two 128-row tiles of one expert, or its last single one)
        self.pair_tiles = torch.empty((self.cap // 128 + E + 1) // 2, 2, dtype=torch.int32, device=dev)
        self.num_pair_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        self.pair = (self.pair_tiles, self.num_pair_tiles)
        # source token of every sorted row (an index outside any tensor for padding rows): operand gathers
        self.row_tok = torch.empty(self.cap, dtype=torch.int32, device=dev)
        scratch = _scratch("moe_plan", e.moe_plan_blocks(n) * E, torch.int32, dev)
        e.moe_plan(idx32.reshape(-1), E, scratch, self.counts, self.seg_off, self.tile_expert, self.num_m_tiles,
                   self.pos, self.row_slot, self.pair_tiles, self.num_pair_tiles, self.row_tok, K)


class MoEExpertsFn(torch.autograd.Function):
    """out[t] = sum_k w[t,k] * down_e(silu(gate_e x_t) * up_e x_t): plan, gather, two grouped GEMMs, combine."""

    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, gate_up, down):
        e = ext()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        T, H = x2.shape
        K = topk_idx.shape[-1]
        w1, w2 = w16(gate_up), w16(down)
        E, I2, _ = w1.shape
        I = I2 // 2
        idx32 = topk_idx.reshape(T, K).to(torch.int32).contiguous()
        tw = topk_w.reshape(T, K).float().contiguous()
        plan = MoEPlan(idx32, E)
        cap, dev = plan.cap, x2.device
        act = torch.empty(cap, I, dtype=BF16, device=dev)
        gu = torch.empty(cap, I2, dtype=BF16, device=dev)
        folded, gathered = G.fold_supported(H, I2), G.gather_supported(H, I2)
        ys = torch.empty(cap, H, dtype=BF16, device=dev)
        out = torch.empty(T, H, dtype=BF16, device=dev)
        if gathered:  # dispatch = the A-operand load: the kernel fetches token rows by index, no sorted copy
            xs, rows = x2, plan.row_tok
        else:
            xs, rows = torch.empty(cap, H, dtype=BF16, device=dev), None
            e.moe_gather(x2, plan.row_slot, plan.seg_off, E, K, xs)
        if folded:
            # The routing weight is applied where the activation is stored, so the combine is a plain sum of K
            # rows and the backward needs neither the expert outputs nor a weighted scatter of the gradient.
            G.grouped_up_swiglu(xs, w1, plan.tile_expert, plan.num_m_tiles, act, gu, pair=plan.pair,
                                gather=rows, row_slot=plan.row_slot, row_w=tw.view(-1))
            G.grouped_nt(act, w2, plan.tile_expert, plan.num_m_tiles, ys, pair=plan.pair)
            e.moe_combine(ys, plan.pos, None, None, out, K, None, 0, None, 0, None)
            ctx.save_for_backward(xs, gu, act, tw)
        else:
            G.grouped_up_swiglu(xs, w1, plan.tile_expert, plan.num_m_tiles, act, gu, pair=plan.pair)
            G.grouped_nt(act, w2, plan.tile_expert, plan.num_m_tiles, ys, pair=plan.pair)
            e.moe_combine(ys, plan.pos, tw, None, out, K, None, 0, None, 0, None)
            ctx.save_for_backward(xs, gu, act, ys, tw)
        ctx.folded = folded
        ctx.gathered = gathered
        ctx.plan = plan
        ctx.params = (gate_up, down)
        ctx.w = (w1, w2)
        ctx.in_shape = tuple(x.shape)
        ctx.counts = plan.counts
        return out.view(ctx.in_shape)

    @staticmethod
    def backward(ctx, dout):
        e = ext()
        plan = ctx.plan
        w1, w2 = ctx.w
        gate_up, down = ctx.params
        T, K, E, cap = plan.T, plan.K, plan.E, plan.cap
        H = ctx.in_shape[-1]
        d2 = dout.reshape(T, H)
        if d2.dtype != BF16:
            d2 = d2.to(BF16)
        d2 = d2.contiguous()
        dev = d2.device
        s2 = GradSink(down)
        t2, b2 = s2.target()
        s1 = GradSink(gate_up)
        t1, b1 = s1.target()
        dx = torch.empty(T, H, dtype=BF16, device=dev)
        if ctx.folded:
            # `act` holds w * silu(g) * u.  d(act) = w * (dout[tok] @ W2) with the SwiGLU backward in the epilogue,
            # which also leaves <dout[tok] @ W2, silu(g) * u> per row and column tile: the routing-weight gradient.
            # With gathered operands the output gradient is read in place by token index; otherwise one unweighted
            # row gather puts it into expert order.
            xs, gu, act, tw = ctx.saved_tensors
            I = act.shape[1]
            rows = plan.row_tok if ctx.gathered else None
            if ctx.gathered:
                dys = d2
                dxs = torch.empty(cap, H, dtype=BF16, device=dev)
            else:
                dys = torch.empty(cap, H, dtype=BF16, device=dev)
                e.moe_gather(d2, plan.row_slot, plan.seg_off, E, K, dys)
                dxs = dys  # reused once the two GEMMs that read it are done
            dgu = torch.empty_like(gu)
            row_dot = torch.empty(cap, (I + 255) // 256, dtype=torch.float32, device=dev)
            G.grouped_nn_swiglu_bwd(dys, w2, plan.tile_expert, plan.num_m_tiles, gu, dgu, pair=plan.pair,
                                    gather=rows, row_slot=plan.row_slot, row_w=tw.view(-1), row_dot=row_dot)
            dw = torch.zeros(T * K, dtype=torch.float32, device=dev)  # slots of dropped rows keep 0
            e.moe_row_dot_reduce(row_dot, plan.row_slot, plan.seg_off, E, dw)
            G.grouped_tn(dys, act, plan.seg_off, t2, beta=b2, a_gather=rows)
            G.grouped_nn(dgu, w1, plan.tile_expert, plan.num_m_tiles, dxs, pair=plan.pair)
            G.grouped_tn(dgu, xs, plan.seg_off, t1, beta=b1, b_gather=rows)
        else:
            xs, gu, act, ys, tw = ctx.saved_tensors
            dys = torch.empty(cap, H, dtype=BF16, device=dev)
            dw = torch.zeros(T * K, dtype=torch.float32, device=dev)
            e.moe_combine_bwd(d2, ys, plan.row_slot, plan.seg_off, tw.view(-1), E, K, dys, dw)
            dgu = torch.empty_like(gu)
            G.grouped_nn_swiglu_bwd(dys, w2, plan.tile_expert, plan.num_m_tiles, gu, dgu, pair=plan.pair)
            G.grouped_tn(dys, act, plan.seg_off, t2, beta=b2)
            dxs = dys  # reuse: dys is dead after the two GEMMs above
            G.grouped_nn(dgu, w1, plan.tile_expert, plan.num_m_tiles, dxs, pair=plan.pair)
            G.grouped_tn(dgu, xs, plan.seg_off, t1, beta=b1)
        e.moe_combine(dxs, plan.pos, None, None, dx, K, None, 0, None, 0, None)
        return dx.view(ctx.in_shape), dw.view(T, K), None, s1.done(t1), s2.done(t2)


def moe_experts(x, topk_idx, topk_w, gate_up, down):
    return MoEExpertsFn.apply(x, topk_w, topk_idx, gate_up, down)


# --------------------------------------------------- fused linear + cross entropy
LCE_CHUNK_ROWS = int(os.environ.get("MOE_B200_LCE_CHUNK", "4096"))
# Measured on a B200 under the power cap: running the memory-bound softmax-gradient pass of chunk c beside the
# vocabulary GEMM of chunk c + 1 does not shorten the sequence (both draw on the same power budget), so the
# second logits buffer it needs is not spent by default.
LCE_OVERLAP = os.environ.get("MOE_B200_LCE_OVERLAP", "0") != "0"
_SIDE_STREAMS: dict = {}


def _side_stream(dev) -> torch.cuda.Stream:
    """One extra stream per device for memory-bound passes that run under a GEMM of the main stream."""
    s = _SIDE_STREAMS.get(dev)
    if s is None:
        s = torch.cuda.Stream(device=dev)
        _SIDE_STREAMS[dev] = s
    return s


class LinearCrossEntropyFn(torch.autograd.Function):
    """Mean cross entropy of `h @ W^T` against aligned labels, without a `[T, V]` tensor.

    Tokens are processed in chunks of `LCE_CHUNK_ROWS` rows that share one reusable bf16 logits scratch
    (`chunk x V`): vocabulary GEMM with softmax partials from its epilogue -> row log-sum-exp and loss ->
    gradient w.r.t. the logits formed in place -> the two gradient GEMMs (dH rows of the chunk; dW
    accumulated over the chunks by the fp32-add epilogue).  Row losses are summed in a fixed order, so the
    loss has the same bits on every run.

    The gradients are produced inside forward, so `upstream` = d(total loss)/d(this loss) must be known
    when forward runs; backward only rescales dH by `dloss / upstream`.  A forward pass under grad mode
    therefore writes into the weight's gradient accumulator even if backward is never called: run
    evaluation passes under `torch.no_grad()`.
    """

    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, upstream):
        e = ext()
        h2 = h.reshape(-1, h.shape[-1])
        if h2.dtype != BF16:
            h2 = h2.to(BF16)
        h2 = h2.contiguous()
        T, H = h2.shape
        dev = h2.device
        wmat = w16(weight)
        V = wmat.shape[0]
        lab = labels.reshape(-1).contiguous()
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        ctx.have_grad = need_grad
        chunk = min(T, max(256, LCE_CHUNK_ROWS))
        n_tiles = (V + 255) // 256
        n_chunks = (T + chunk - 1) // chunk
        # two logits buffers when there is more than one chunk: the memory-bound softmax-gradient pass of
        # chunk c runs on a side stream under the (compute-bound) vocabulary GEMM of chunk c + 1
        overlap = need_grad and n_chunks > 1 and LCE_OVERLAP
        nbuf = 2 if overlap else 1
        logits_bufs = [_scratch(f"lce_logits{i}", chunk * V, BF16, dev) for i in range(nbuf)]
        part_buf = _scratch("lce_part", chunk * n_tiles * 2, torch.float32, dev)
        lse = torch.empty(T, dtype=torch.float32, device=dev)
        row_loss = torch.empty(T, dtype=torch.float32, device=dev)
        acc = torch.empty(3, dtype=torch.float32, device=dev)
        e.lce_reduce(None, lab, ignore_index, V, acc)  # number of valid labels, needed by every gradient tile
        if need_grad:
            dh = torch.empty(T, H, dtype=BF16, device=dev)
            sink = GradSink(weight)
            tgt, beta = sink.target()
        main = torch.cuda.current_stream(dev)
        side = _side_stream(dev) if overlap else None
        spans = [(c0, min(chunk, T - c0)) for c0 in range(0, T, chunk)]

        def logits_of(i):
            return logits_bufs[i % nbuf][:spans[i][1] * V].view(spans[i][1], V)

        def front(i):  # vocabulary GEMM + row statistics (+ gradient w.r.t. the logits, in place)
            c0, rows = spans[i]
            logits = logits_of(i)
            part = part_buf[:rows * n_tiles * 2].view(rows, n_tiles, 2)
            G.gemm_nt_lse(h2[c0:c0 + rows], wmat, logits, part)
            e.lse_loss(part, logits, lab[c0:c0 + rows], ignore_index, lse[c0:c0 + rows], row_loss[c0:c0 + rows])
            if not need_grad:
                return None
            if side is None:
                e.dlogits_(logits, lse[c0:c0 + rows], lab[c0:c0 + rows], ignore_index, acc, float(upstream))
                return None
            ready = torch.cuda.Event()
            ready.record(main)
            done = torch.cuda.Event()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                e.dlogits_(logits, lse[c0:c0 + rows], lab[c0:c0 + rows], ignore_index, acc, float(upstream))
                done.record(side)
            return done

        def back(i, done):  # the two gradient GEMMs of chunk i
            c0, rows = spans[i]
            if done is not None:
                main.wait_event(done)
            logits = logits_of(i)
            G.gemm_nn(logits, wmat, out=dh[c0:c0 + rows], m_fast=0)
            G.gemm_tn(logits, h2[c0:c0 + rows], tgt, beta=beta if i == 0 else 1)

        pending = None
        for i in range(n_chunks):
            done = front(i)
            if need_grad:
                if overlap:
                    if pending is not None:
                        back(*pending)
                    pending = (i, done)
                else:
                    back(i, done)
        if pending is not None:
            back(*pending)
        e.lce_reduce(row_loss, lab, ignore_index, V, acc)
        if need_grad:
            ctx.dw = sink.done(tgt)
            ctx.save_for_backward(dh)
            ctx.in_shape = tuple(h.shape)
            ctx.upstream = float(upstream)
        return acc[2]

    @staticmethod
    def backward(ctx, dloss):
        if not ctx.have_grad:
            return None, None, None, None, None
        (dh,) = ctx.saved_tensors
        dw = ctx.dw
        ctx.dw = None
        dh = dh * (dloss / ctx.upstream).to(dh.dtype)
        return dh.view(ctx.in_shape), dw, None, None, None


def linear_cross_entropy(h, weight, labels, ignore_index=-100, upstream=1.0):
    return LinearCrossEntropyFn.apply(h, weight, labels, ignore_index, upstream)
