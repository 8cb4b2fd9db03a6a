"""Load-balancing losses in histogram form.

Same values as the reference (`src/models/load_balancing.py:19-169`) without ever building a
`[N, K, E]` one-hot tensor: the hard assignment enters only through per-expert counts.

* Switch loss: `aux = E * sum_e (cnt_e / N) * (sum_t p_te / N)` over all layers pooled, `cnt`
  from the unbiased top-k of the recorded scores, statistics local to the rank, gradient
  through `p` only.  Uniform routing gives `aux = top_k`.
* DeepSeek-V3 sequence-level loss (arXiv 2412.19437, Eq. 17-20), per sequence, averaged over
  sequences and layers.  Uniform routing gives 1.
"""
from __future__ import annotations

import torch

from ..ops.oracle import topk_lowest_index


def _counts(idx: torch.Tensor, num_experts: int, weight: torch.Tensor | None = None) -> torch.Tensor:
    flat = idx.reshape(-1).long()
    src = torch.ones(flat.numel(), dtype=torch.float32, device=idx.device) if weight is None else weight
    return torch.zeros(num_experts, dtype=torch.float32, device=idx.device).index_add_(0, flat, src)


def load_balancing_loss_func(gate_logits, num_experts: int | None = None, top_k: int = 2,
                             attention_mask: torch.Tensor | None = None, selected_experts=None):
    """Switch-Transformer auxiliary loss on router *probabilities* (no second softmax).

    `gate_logits`: tuple of per-layer `[T, E]` score tensors.  `selected_experts` (optional tuple of
    `[T, K]` index tensors) skips the top-k when the caller already has the unbiased selection.
    """
    if gate_logits is None or not isinstance(gate_logits, tuple):
        return 0
    dev = gate_logits[0].device
    E = num_experts if num_experts is not None else gate_logits[0].shape[-1]
    cnt = torch.zeros(E, dtype=torch.float32, device=dev)
    psum = torch.zeros(E, dtype=torch.float32, device=dev)
    n_total = 0.0
    tok_w = None
    if attention_mask is not None:
        tok_w = attention_mask.reshape(-1).to(device=dev, dtype=torch.float32)
    for li, probs in enumerate(gate_logits):
        probs = probs.to(dev)
        pf = probs.float()
        if selected_experts is not None and selected_experts[li] is not None:
            idx = selected_experts[li]
        else:
            _, idx = topk_lowest_index(pf.detach(), top_k)
        if tok_w is None:
            cnt = cnt + _counts(idx, E)
            psum = psum + pf.sum(dim=0)
            n_total += pf.shape[0]
        else:
            wk = tok_w.repeat_interleave(idx.shape[-1])
            cnt = cnt + _counts(idx, E, wk)
            psum = psum + (pf * tok_w[:, None]).sum(dim=0)
            n_total = n_total + tok_w.sum()
    f = cnt / n_total
    p = psum / n_total
    return (f * p).sum() * E


def seq_load_balancing_loss_func(gate_logits, num_experts: int | None = None, top_k: int = 2, batch_size: int = 1,
                                 selected_experts=None):
    """Sequence-level balance loss; `selected_experts` = the routers' actual (biased) choices."""
    if gate_logits is None or not isinstance(gate_logits, tuple):
        return 0
    total = gate_logits[0].new_zeros((), dtype=torch.float32)
    for li, layer_gate in enumerate(gate_logits):
        T, E = layer_gate.shape
        S = T // batch_size
        s = layer_gate.float()
        s = s / (s.sum(dim=-1, keepdim=True) + 1e-20)
        s = s.reshape(batch_size, S, E)
        sel = None
        if selected_experts is not None and li < len(selected_experts):
            cand = selected_experts[li]
            if cand is not None and tuple(cand.shape) == (T, top_k):
                sel = cand.reshape(batch_size, S * top_k).to(s.device).long()
        if sel is None:
            sel = topk_lowest_index(s.detach(), top_k)[1].reshape(batch_size, S * top_k)
        counts = torch.zeros(batch_size, E, dtype=torch.float32, device=s.device)
        counts.scatter_add_(1, sel, torch.ones_like(sel, dtype=torch.float32))
        f = counts * (E / (top_k * S))
        P = s.mean(dim=1)
        total = total + (f * P).sum(dim=-1).mean()
    return total / len(gate_logits)
