"""Plain-PyTorch statement of every op in the model.

This module is both the CPU execution path (fp32, differentiable through
ordinary autograd) and the numerical oracle for the sm_100a kernels.
Semantics follow the Qwen3-MoE backbone the reference inherits
(`src/models/modeling_qwen3_moe.py:56-307`) and its router / loss code
(`src/models/router.py:22-155`, `src/models/load_balancing.py:19-169`).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """fp32 `x * rsqrt(mean(x^2) + eps)`, cast to the input dtype, then times weight."""
    dt = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = (xf * torch.rsqrt(var + eps)).to(dt)
    return weight.to(dt) * y


# ---------------------------------------------------------------------- RoPE
def rope_tables(seq_len: int, head_dim: int, theta: float, device=None, offset: int = 0
                ) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables `[seq_len, head_dim]` in fp32 (`emb = cat(freqs, freqs)`)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    pos = torch.arange(offset, offset + seq_len, dtype=torch.float32, device=device)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: `[B, S, heads, hd]`; cos/sin: `[S, hd]`."""
    c = cos.to(x.dtype)[None, :, None, :]
    s = sin.to(x.dtype)[None, :, None, :]
    return x * c + rotate_half(x) * s


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                 cos: torch.Tensor, sin: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-head RMSNorm over head_dim (weight shared by all heads) followed by RoPE."""
    return apply_rope(rmsnorm(q, q_weight, eps), cos, sin), apply_rope(rmsnorm(k, k_weight, eps), cos, sin)


# ----------------------------------------------------------------- attention
def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None
                         ) -> torch.Tensor:
    """q `[B,S,nh,hd]`, k/v `[B,S,nkv,hd]` -> `[B,S,nh,hd]`; fp32 softmax, causal."""
    B, S, nh, hd = q.shape
    nkv = k.shape[2]
    g = nh // nkv
    scale = hd ** -0.5 if scale is None else scale
    qh = q.transpose(1, 2)
    kh = k.transpose(1, 2).repeat_interleave(g, dim=1)
    vh = v.transpose(1, 2).repeat_interleave(g, dim=1)
    att = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1)
    att = att.masked_fill(mask, float("-inf"))
    att = torch.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.matmul(att, vh).transpose(1, 2).contiguous()


# ------------------------------------------------------------------- routing
def topk_lowest_index(scores: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k along the last dim; ties go to the lowest index (stable descending sort)."""
    vals, idx = torch.sort(scores, dim=-1, descending=True, stable=True)
    return vals[..., :k], idx[..., :k]


def group_limited_topk(scores: torch.Tensor, topk: int, num_groups: int, group_topk: int
                       ) -> tuple[torch.Tensor, torch.Tensor]:
    """Group-limited routing (`src/models/router.py:22-70`): score each group by the sum of its
    top-(topk // group_topk) entries, keep `group_topk` groups, then take top-k inside them."""
    T, E = scores.shape
    per = E // num_groups
    grouped = scores.view(T, num_groups, per)
    group_scores = topk_lowest_index(grouped, topk // group_topk)[0].sum(-1)
    gidx = topk_lowest_index(group_scores, group_topk)[1]
    gmask = torch.zeros_like(group_scores, dtype=torch.bool).scatter_(1, gidx, True)
    emask = gmask.unsqueeze(-1).expand(T, num_groups, per).reshape(T, E)
    masked = scores.masked_fill(~emask, float("-inf"))
    return topk_lowest_index(masked, topk)


def router_softmax(x: torch.Tensor, weight: torch.Tensor, top_k: int, norm_topk_prob: bool
                   ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Softmax router: returns (probs fp32 [T,E], weights fp32 [T,K], indices int64 [T,K])."""
    logits = F.linear(x.float(), weight.float())
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    w, idx = topk_lowest_index(probs, top_k)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return probs, w, idx


def router_sigmoid(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, top_k: int,
                   norm_topk_prob: bool, scaling_factor: float | None, num_groups: int | None,
                   group_topk: int | None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sigmoid router with a selection-only bias (`src/models/router.py:103-155`)."""
    scores = torch.sigmoid(F.linear(x.float(), weight.float()))
    biased = scores if bias is None else scores + bias.float().unsqueeze(0)
    if num_groups is not None and group_topk is not None:
        _, idx = group_limited_topk(biased.detach(), top_k, num_groups, group_topk)
    else:
        _, idx = topk_lowest_index(biased.detach(), top_k)
    w = scores.gather(1, idx)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    if scaling_factor is not None:
        w = w * scaling_factor
    return scores, w, idx


# ------------------------------------------------------------------- experts
def moe_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor
                ) -> torch.Tensor:
    """`out[t] = sum_k w[t,k] * down_e(silu(gate_e x_t) * up_e x_t)`, e = idx[t,k].

    `gate_up [E, 2I, H]` (gate rows first), `down [E, H, I]`
    (`src/models/modeling_qwen3_moe.py:217-254`).  Experts with no token are skipped.
    """
    T, H = x.shape
    E = gate_up.shape[0]
    out = torch.zeros_like(x)
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    counts = torch.bincount(flat_e, minlength=E).tolist()
    tok = order // idx.shape[1]
    wk = w.reshape(-1)[order].to(x.dtype)
    start = 0
    for e in range(E):
        c = counts[e]
        if c == 0:
            continue
        t_e = tok[start:start + c]
        xe = x[t_e]
        g, u = F.linear(xe, gate_up[e].to(x.dtype)).chunk(2, dim=-1)
        ye = F.linear(F.silu(g) * u, down[e].to(x.dtype)) * wk[start:start + c, None]
        out.index_add_(0, t_e, ye)
        start += c
    return out


def swiglu_mlp(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    return F.linear(F.silu(F.linear(x, gate_w)) * F.linear(x, up_w), down_w)


# ---------------------------------------------------------------------- loss
def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100
                         ) -> torch.Tensor:
    """Mean token cross entropy of `h @ weight^T` against `labels` (already aligned with `h`)."""
    logits = F.linear(h, weight.to(h.dtype)).float()
    return F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="mean")


def shift_labels(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Position t predicts token t+1; the last position of every sequence is ignored."""
    out = torch.full_like(labels, ignore_index)
    out[..., :-1] = labels[..., 1:]
    return out


# ----------------------------------------------------------------- optimiser
def adamw_step_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float,
                beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0) -> None:
    """One decoupled-weight-decay Adam update in place (same arithmetic as `torch.optim.AdamW`)."""
    g = g * grad_scale if grad_scale != 1.0 else g
    p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
