"""Op layer: every model op has a plain-PyTorch statement (`oracle`, CPU / fp32) and an
sm_100a kernel path (`functional`, CUDA / bf16).  Dispatch is by device: CUDA tensors always
take the kernel path and fail loudly if the extension is missing."""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from . import oracle

_FORCE_ORACLE = False


class force_oracle:
    """Context manager: run CUDA tensors through the plain-PyTorch ops (for kernel-vs-oracle tests)."""

    def __enter__(self):
        global _FORCE_ORACLE
        self.prev = _FORCE_ORACLE
        _FORCE_ORACLE = True

    def __exit__(self, *a):
        global _FORCE_ORACLE
        _FORCE_ORACLE = self.prev


def _k(x: torch.Tensor) -> bool:
    return x.is_cuda and not _FORCE_ORACLE


def _f():
    from . import functional

    return functional


def embedding(ids, weight):
    if _k(weight):
        return _f().EmbeddingFn.apply(ids, weight)
    return TF.embedding(ids, weight)


def rmsnorm(x, weight, eps):
    if _k(x):
        return _f().rmsnorm(x, weight, eps)
    return oracle.rmsnorm(x, weight, eps)


def add_rmsnorm(x, res, weight, eps):
    """Returns (x + res, rmsnorm(x + res))."""
    if _k(x):
        return _f().add_rmsnorm(x, res, weight, eps)
    h = x + res
    return h, oracle.rmsnorm(h, weight, eps)


def linear(x, *weights, fused=None):
    """x @ cat(weights)^T (weights are row blocks of one matrix)."""
    if _k(x):
        return _f().linear(x, *weights, fused=fused)
    w = weights[0] if len(weights) == 1 else torch.cat(list(weights), dim=0)
    return TF.linear(x, w.to(x.dtype))


def qk_norm_rope(qkv, q_w, k_w, B, S, nh, nkv, hd, theta, eps):
    """Split a fused QKV activation and apply per-head RMSNorm + RoPE to q and k; `[B,S,h,hd]` outputs."""
    if _k(qkv):
        return _f().qk_norm_rope(qkv, q_w, k_w, B, S, nh, nkv, hd, theta, eps)
    q, k, v = qkv.view(B, S, nh + 2 * nkv, hd).split([nh, nkv, nkv], dim=2)
    cos, sin = oracle.rope_tables(S, hd, theta, device=qkv.device)
    q, k = oracle.qk_norm_rope(q, k, q_w, k_w, cos, sin, eps)
    return q, k, v


def qkv_proj_norm_rope(x, wq, wk, wv, fused, q_norm_w, k_norm_w, B, S, nh, nkv, hd, theta, eps):
    """Hidden states -> (q, k, v) `[B,S,h,hd]`: QKV projection, per-head RMSNorm of q and k, RoPE."""
    if _k(x):
        return _f().qkv_proj_norm_rope(x, wq, wk, wv, fused, q_norm_w, k_norm_w, B, S, nh, nkv, hd, theta, eps)
    qkv = linear(x, wq, wk, wv, fused=fused)
    return qk_norm_rope(qkv, q_norm_w, k_norm_w, B, S, nh, nkv, hd, theta, eps)


def attention(q, k, v):
    if _k(q):
        return _f().attention(q, k, v)
    return oracle.causal_gqa_attention(q, k, v)


def kernel_path(x: torch.Tensor) -> bool:
    """True when ops on `x` run the sm_100a kernels (CUDA tensor, oracle not forced)."""
    return _k(x)


def router(x, weight, bias, *, top_k, score_fn, norm_topk_prob, scaling_factor, num_groups, group_topk, site=None,
           tokens_acc=None, collect=True):
    """Returns (scores fp32 [T,E], weights fp32 [T,K], indices [T,K]).  Kernel path only: `site` (a
    `functional.RouterSite`) receives the routing statistics of this call, `tokens_acc` the selection counts;
    `collect=False` (recomputation of a checkpointed layer) leaves both untouched."""
    if _k(x):
        mode = 0 if score_fn == "softmax" else 1
        return _f().router(x, weight, bias, top_k, mode, norm_topk_prob, scaling_factor, num_groups, group_topk,
                           site, tokens_acc, collect)
    if score_fn == "softmax" and bias is None and num_groups is None:
        s, w, i = oracle.router_softmax(x, weight, top_k, norm_topk_prob)
        if scaling_factor is not None:
            w = w * scaling_factor
        return s, w, i
    if score_fn == "softmax":
        probs = torch.softmax(TF.linear(x.float(), weight.float()), dim=-1, dtype=torch.float32)
        biased = probs if bias is None else probs + bias.float()
        if num_groups is not None:
            _, idx = oracle.group_limited_topk(biased.detach(), top_k, num_groups, group_topk)
        else:
            _, idx = oracle.topk_lowest_index(biased.detach(), top_k)
        w = probs.gather(1, idx)
        if norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        if scaling_factor is not None:
            w = w * scaling_factor
        return probs, w, idx
    return oracle.router_sigmoid(x, weight, bias, top_k, norm_topk_prob, scaling_factor, num_groups, group_topk)


def moe_aux_losses(holder, scores, seq_on: bool):
    """(Switch loss, sequence-level loss) from the statistics the router kernels wrote into `holder`."""
    return _f().moe_aux_losses(holder, scores, seq_on)


def set_moe_site(mlp, global_experts, layer_idx: int) -> None:
    """Tell the expert-parallel context (if any) which decoder layer is about to call `moe_experts`."""
    bank = global_experts if global_experts is not None else getattr(mlp, "experts", None)
    ep = getattr(getattr(bank, "gate_up_proj", None), "_ep", None)
    if ep is not None:
        ep.site = layer_idx


def moe_experts(x, idx, w, gate_up, down):
    ep = getattr(gate_up, "_ep", None)
    if ep is not None:  # experts sharded over ranks: dispatch / combine over NVLink peer memory
        from ..parallel.ep import moe_experts_ep

        return moe_experts_ep(x, idx, w, gate_up, down, ep)
    if getattr(gate_up, "_ep_shard", None) is not None:
        raise RuntimeError("expert-parallel parameters need an EPContext (create the model through Trainer)")
    if _k(x):
        return _f().moe_experts(x, idx, w, gate_up, down)
    return oracle.moe_experts(x, idx.long(), w, gate_up, down)


def swiglu_mlp(x, gate_w, up_w, down_w, fused_gate_up=None):
    if _k(x):
        return _f().swiglu_mlp(x, gate_w, up_w, down_w, fused_gate_up)
    return oracle.swiglu_mlp(x, gate_w.to(x.dtype), up_w.to(x.dtype), down_w.to(x.dtype))


def linear_cross_entropy(h, weight, labels, ignore_index=-100, upstream=1.0):
    """Mean cross entropy of h @ weight^T; labels are already aligned with h (no shift here)."""
    if _k(h):
        return _f().linear_cross_entropy(h, weight, labels, ignore_index, upstream)
    return oracle.linear_cross_entropy(h.reshape(-1, h.shape[-1]), weight, labels.reshape(-1), ignore_index)
