"""Causal-LM heads over the decoder: the five model types of the reference.

Call convention follows the reference models (`src/models/standard_moe.py:20-66`,
`src/models/global_moe.py:154-213`): keyword-only `model(input_ids=..., labels=...,
output_router_logits=True)` returning an object with `.loss`, `.aux_loss`, `.logits`,
`.router_logits`.  `loss = ce + router_aux_loss_coef * aux + _seq_aux_loss_coef * seq_aux`.
Labels are shifted once, inside the model (position t predicts token t+1).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..ops.oracle import shift_labels
from ..utils.profiling import phase
from .backbone import DecoderModel, Linear, init_weights_
from .config import GlobalMoEConfig, Qwen3Config, Qwen3MoeConfig
from .load_balancing import load_balancing_loss_func, seq_load_balancing_loss_func
from .router import DeepSeekRouter, TopKRouter


class MoeCausalLMOutput:
    """Attribute bag (also indexable by key) for model outputs."""

    def __init__(self, **kw):
        self.loss = None
        self.aux_loss = None
        self.logits = None
        self.router_logits = None
        self.ce_loss = None
        self.seq_aux_loss = None
        self.hidden_states = None
        self.router_stats = None  # kernel path: the `MoeStatsHolder` with this pass's routing statistics
        self.__dict__.update(kw)

    def __getitem__(self, k):
        return getattr(self, k)

    def get(self, k, default=None):
        return getattr(self, k, default)


class GlobalMoEModel(DecoderModel):
    """Decoder whose layers all route into one shared expert bank (`model.global_experts`)."""

    def __init__(self, config: GlobalMoEConfig, router_class=None):
        super().__init__(config, "global", router_class)


class _CausalLM(nn.Module):
    layout = "standard"
    _router_class = None
    is_moe = True

    def __init__(self, config, seed: int | None = None):
        super().__init__()
        self.config = config
        if self.layout == "global":
            self.model = GlobalMoEModel(config, router_class=self._router_class)
        else:
            self.model = DecoderModel(config, self.layout, router_class=self._router_class)
        self.vocab_size = config.vocab_size
        self.lm_head = Linear(config.hidden_size, config.vocab_size)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.router_aux_loss_coef = getattr(config, "router_aux_loss_coef", 0.0)
        self.num_experts = getattr(config, "num_experts", 0)
        self.num_experts_per_tok = getattr(config, "num_experts_per_tok", 0)
        self._seq_aux_loss_coef = 0.0
        self.post_init(seed)

    # ---- HF-compatible odds and ends used by the reference's train.py / scripts
    def post_init(self, seed: int | None = None):
        gen = None
        if seed is not None:
            dev = next(self.parameters()).device
            gen = torch.Generator(device=dev if dev.type == "cuda" else "cpu")
            gen.manual_seed(seed)
        init_weights_(self, std=getattr(self.config, "initializer_range", 0.02), generator=gen)

    def set_experts_implementation(self, name: str) -> None:
        """Accepted for compatibility; there is a single expert path per device."""
        self._experts_implementation = name

    def gradient_checkpointing_enable(self, *a, **k) -> None:
        self.model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self) -> None:
        self.model.gradient_checkpointing = False

    def routers(self):
        return [layer.mlp.gate for layer in self.model.layers if hasattr(layer.mlp, "gate")]

    # ---- forward
    def forward(self, **kwargs):
        input_ids = kwargs.get("input_ids")
        labels = kwargs.get("labels")
        attention_mask = kwargs.get("attention_mask")
        want_router = kwargs.get("output_router_logits")
        if want_router is None:
            want_router = getattr(self.config, "output_router_logits", False)
        loss_scale = float(kwargs.get("loss_scale", 1.0))
        if input_ids is None:
            raise ValueError("input_ids is required")
        holder = self._begin_stats(input_ids, attention_mask) if (self.is_moe and want_router) else None
        if holder is None and self.is_moe:
            for r in self.routers():
                r._site = None
        # (the sites stay attached after the call: a checkpointed layer is recomputed during backward)
        hidden, scores = self.model(input_ids)
        out = MoeCausalLMOutput()
        if kwargs.get("output_hidden_states"):
            out.hidden_states = hidden
        if labels is not None:
            tgt = shift_labels(labels)
            with phase("lce"):
                ce = ops.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), self.lm_head.weight,
                                              tgt.reshape(-1), -100, loss_scale)
            out.ce_loss = ce
            out.loss = ce
        if labels is None or kwargs.get("return_logits"):
            out.logits = ops.linear(hidden, self.lm_head.weight)
        if self.is_moe and want_router and len(scores) > 0 and holder is not None:
            # kernel path: both losses come from the statistics the router kernels left behind
            out.router_logits = scores
            out.router_stats = holder
            seq_coef = getattr(self, "_seq_aux_loss_coef", 0.0)
            aux, seq_aux = ops.moe_aux_losses(holder, scores, seq_on=seq_coef > 0)
            out.aux_loss = aux
            if out.loss is not None:
                out.loss = out.loss + self.router_aux_loss_coef * aux
                if seq_coef > 0:
                    out.seq_aux_loss = seq_aux
                    out.loss = out.loss + seq_coef * seq_aux
        elif self.is_moe and want_router and len(scores) > 0:
            out.router_logits = scores
            sel_unbiased = None
            routers = self.routers()
            if all((not r.use_bias) and r.num_groups is None for r in routers):
                sel_unbiased = tuple(r._last_top_k_idx for r in routers)
            aux = load_balancing_loss_func(scores, self.num_experts, self.num_experts_per_tok, attention_mask,
                                           selected_experts=sel_unbiased)
            out.aux_loss = aux
            if out.loss is not None:
                out.loss = out.loss + self.router_aux_loss_coef * aux
            seq_coef = getattr(self, "_seq_aux_loss_coef", 0.0)
            if seq_coef > 0 and out.loss is not None:
                selected = tuple(r._last_top_k_idx for r in routers)
                seq_aux = seq_load_balancing_loss_func(scores, self.num_experts, self.num_experts_per_tok,
                                                       batch_size=input_ids.shape[0], selected_experts=selected)
                out.seq_aux_loss = seq_aux
                out.loss = out.loss + seq_coef * seq_aux
        return out

    def _begin_stats(self, input_ids, attention_mask):
        """Kernel path only: hand every router its slot of the stacked statistics buffers."""
        weight = self.model.embed_tokens.weight
        if attention_mask is not None or not ops.kernel_path(weight) or input_ids.dim() != 2:
            return None
        routers = self.routers()
        if not routers:
            return None
        from ..ops.functional import MoeStatsHolder

        B, S = input_ids.shape
        key = (B, S, weight.device)
        cache = self.__dict__.setdefault("_stats_holders", {})
        holder = cache.get(key)
        if holder is None:
            holder = MoeStatsHolder(len(routers), B, S, self.num_experts, self.num_experts_per_tok, weight.device,
                                    any(r.separate_unbiased() for r in routers))
            cache[key] = holder
        holder.begin()
        for r, site in zip(routers, holder.sites):
            r._site = site
        return holder

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 16, temperature: float = 0.0,
                 generator: torch.Generator | None = None) -> torch.Tensor:
        """Plain autoregressive sampling without a KV cache (sanity sampling only)."""
        was = self.training
        self.eval()
        ids = input_ids
        for _ in range(max_new_tokens):
            logits = self(input_ids=ids, output_router_logits=False).logits[:, -1].float()
            if temperature and temperature > 0:
                nxt = torch.multinomial(torch.softmax(logits / temperature, -1), 1, generator=generator)
            else:
                nxt = logits.argmax(-1, keepdim=True)
            ids = torch.cat([ids, nxt], dim=1)
        self.train(was)
        return ids


class StandardMoEModel(_CausalLM):
    """Every layer owns `num_experts` experts; softmax top-k router."""

    layout = "standard"


class DeepSeekStandardMoEModel(StandardMoEModel):
    """Standard layout with the sigmoid + expert-bias router."""

    _router_class = DeepSeekRouter


class GlobalMoEForCausalLM(_CausalLM):
    """One bank of `num_experts` experts shared by all layers, per-layer routers."""

    layout = "global"


class DeepSeekGlobalMoEForCausalLM(GlobalMoEForCausalLM):
    _router_class = DeepSeekRouter


class Qwen3ForCausalLM(_CausalLM):
    """Dense SwiGLU baseline."""

    layout = "dense"
    is_moe = False


Qwen3MoeForCausalLM = StandardMoEModel

__all__ = ["MoeCausalLMOutput", "StandardMoEModel", "DeepSeekStandardMoEModel", "GlobalMoEModel",
           "GlobalMoEForCausalLM", "DeepSeekGlobalMoEForCausalLM", "Qwen3ForCausalLM", "Qwen3MoeForCausalLM",
           "TopKRouter", "DeepSeekRouter", "Qwen3Config", "Qwen3MoeConfig", "GlobalMoEConfig"]
